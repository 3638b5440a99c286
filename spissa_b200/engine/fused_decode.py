"""A decode step's layers in one persistent kernel, when every layer's parts allow it.

The parts stay what decides: each may describe itself through ``fused_fields()`` (tensors, sizes and
constants, see ``parts.base.Part``). If every entry of the schedule is a pre-norm block of an RMS norm, a
rotary grouped-query attention that writes its own cache and a SwiGLU feed-forward, in bfloat16, the layers of
a step that brings one token per sequence (up to 16 sequences) run as ``csrc/decode_layers.cu``; any other
model, step or size runs part by part as before. Both ways give the same result up to rounding and are
compared with each other and with the plain implementation in the tests.
"""
from __future__ import annotations

import os
import struct

import torch

from ..csrc import lib as K

MAX_TOKENS = 16


def five_launch_from(layer_bytes: float) -> int:
    """The number of sequences from which a decode step is faster as the five-launch sequence of the weight-streaming
    tcgen05 product (``engine/fused_prefill.py``) than in this kernel, by the bytes of a layer's weights. Measured on a
    B200, decode step in ms, this kernel / five launches:

        1B layers, 122 MB (width 2048, head 64):   8 sequences 0.95 / 1.14,  16: 1.09 / 1.37
        3B layers, 201 MB (width 3072, head 128):  2: 2.21 / 2.08,  4: 2.32 / 2.26,  6: 2.44 / 2.35,  8: 2.57 / 2.38,
                                                   12: 2.87 / 2.73,  16: 3.06 / 2.87
        8B layers, 436 MB (width 4096, head 128):  4: 3.93 / 4.01,  6: 4.11 / 4.15,  7: 4.30 / 4.39,  8: 4.7 / 4.21,
                                                   9: 4.54 / 4.45,  12: 5.17 / 4.84,  16: 6.4 / 5.06

    The kernel's products walk blocks of 16 rows dealt to 148 CTAs; the 3B widths leave many CTAs a round short (192
    blocks: two rounds for 44 of them), and with more than 8 tokens it keeps 16 rows of normed activations in shared
    memory (128 KB at width 4096: two ring stages are left of four) and one tile's fragments in flight instead of two.
    """
    if layer_bytes <= 160e6:
        return MAX_TOKENS + 1                  # never
    if layer_bytes <= 300e6:
        return 2
    return 8


def collect_fused_fields(model):
    """Per schedule entry what the blocks say of themselves through ``fused_fields()``, when every entry is a
    pre-norm block of an RMS norm, a rotary grouped-query attention that writes its own cache and a SwiGLU, all
    bfloat16 and of one width and head size; else None. Shared by the one-kernel decode path and the fused prompt path."""
    if model.rt is None or model.rt.act_dtype != torch.bfloat16 or not model.spec.schedule:
        return None
    fields = []
    for e in model.spec.schedule:
        blk = model.layers[e.layer]
        f = blk.fused_fields() if e.writes_cache else None
        if not f or f.get("kind") != "prenorm" or f["mixer"].get("kind") != "gqa_rotary" \
                or f["ffn"].get("kind") != "swiglu" or f["mixer_norm"].get("kind") != "rmsnorm" \
                or f["ffn_norm"].get("kind") != "rmsnorm":
            return None
        fields.append(f)
    H, hd = fields[0]["mixer"]["hidden_size"], fields[0]["mixer"]["head_dim"]
    for f in fields:
        m, ff = f["mixer"], f["ffn"]
        if m["hidden_size"] != H or m["head_dim"] != hd or ff["hidden_size"] != H:
            return None
        if f["mixer_norm"]["size"] != H or f["ffn_norm"]["size"] != H:
            return None
        if ff["pair"] % 8 or ff["intermediate_size"] % 8 or (m["num_heads"] * hd) % 8 or H % 16:
            return None
        for w in (m["qkv"], m["o"], ff["gate_up"], ff["down"]):
            if not w.is_contiguous() or w.data_ptr() % 16:
                return None
    return fields


class FusedDecode:
    """The descriptor table and scratch buffers of one model on one cache."""

    def __init__(self, model, fields: list):
        self.model = model
        self.fields = fields                   # per schedule entry
        first = fields[0]["mixer"]
        self.H = first["hidden_size"]
        self.hd = first["head_dim"]
        self.max_nkv = max(f["mixer"]["num_kv_heads"] for f in fields)
        self.max_nh = max(f["mixer"]["num_heads"] for f in fields)
        self.max_group = max(f["mixer"]["num_heads"] // f["mixer"]["num_kv_heads"] for f in fields)
        self.max_I = max(f["ffn"]["intermediate_size"] for f in fields)
        # bytes of the largest layer's weights: decides from how many sequences on another runner is faster
        self.layer_bytes = max(sum(w.numel() * w.element_size() for w in (f["mixer"]["qkv"], f["mixer"]["o"], f["ffn"]["gate_up"],
                                                                     f["ffn"]["down"])) for f in fields)
        self.table = None
        self.runs = 0                          # steps run through the kernel so far
        self.cache_id = None
        self.group = None
        self._splits = {}                      # (sequences, pages) -> the kernel's split of the keys
        self.head = None                       # the final norm and the head, when the kernel can take them too
        # switch for comparisons: False (or SPISSA_B200_FUSE_HEAD=0) leaves the final norm and the head to the parts
        self.with_head = os.environ.get("SPISSA_B200_FUSE_HEAD", "1") != "0"
        self.head_runs = 0
        self.embedding = None                  # the embedding table, when the kernel can gather the rows itself

    # ------------------------------------------------------------------ planning
    @classmethod
    def plan(cls, model):
        """A runner for ``model`` or None when some layer has to run part by part."""
        fields = collect_fused_fields(model)
        if fields is None:
            return None
        H, hd = fields[0]["mixer"]["hidden_size"], fields[0]["mixer"]["head_dim"]
        plan = cls(model, fields)
        if not K.decode_layers_supported(1, H, hd, model.rt.page_size, plan.max_group):
            return None
        # the final norm and the head as the kernel's last product, when they say what they are
        norm = model.final_norm.fused_fields() if hasattr(model.final_norm, "fused_fields") else None
        head = model.head.fused_fields() if hasattr(model.head, "fused_fields") else None
        if norm and head and norm.get("kind") == "rmsnorm" and head.get("kind") == "linear_head" \
                and norm["size"] == H and head["hidden_size"] == H and head["vocab_size"] % 16 == 0:
            plan.head = dict(weight=head["weight"], norm=norm["weight"], eps=float(norm["eps"]), vocab=head["vocab_size"])
        emb = model.embedding.fused_fields() if hasattr(model.embedding, "fused_fields") else None
        if emb and emb.get("kind") == "token_embedding" and emb["hidden_size"] == H:
            plan.embedding = emb["weight"]
        return plan

    def takes(self, step, cache) -> bool:
        return step.all_single and self.takes_sizes(step.n_tokens, step.max_len, cache)

    def takes_sizes(self, n_seqs: int, max_len: int, cache) -> bool:
        """Whether a decode step of ``n_seqs`` sequences, the longest of ``max_len`` tokens, goes through the kernel."""
        if n_seqs > MAX_TOKENS:
            return False
        if n_seqs >= five_launch_from(self.layer_bytes) and self._five_launch() is not None:
            return False                               # faster as five launches a layer: see five_launch_from
        if (max_len + cache.page_size - 1) // cache.page_size > K.decode_layers_max_pages():
            return False
        if not K.decode_layers_supported(n_seqs, self.H, self.hd, cache.page_size, self.max_group):
            return False
        if self.cache_id != id(cache):
            self._bind_cache(cache)
        return self.table is not None

    def _five_launch(self):
        """The runner of the five-launch sequence for this model, if there is one."""
        m = self.model
        if not m.fuse_prefill:
            return None
        if m._fused_prefill is False:
            from .fused_prefill import FusedPrefill
            m._fused_prefill = FusedPrefill.plan(m)
        return m._fused_prefill

    def key_split(self, n_seqs: int, max_len: int, page_size: int) -> tuple:
        """(pages per chunk, chunks) for a step: what a captured launch reads from the device before it runs."""
        key = (n_seqs, (max_len + page_size - 1) // page_size)
        got = self._splits.get(key)
        if got is None:
            if len(self._splits) > 4096:
                self._splits.clear()
            got = self._splits[key] = K.decode_layers_plan(n_seqs, self.hd, key[1], self.max_nkv)
        return got

    def _bind_cache(self, cache) -> None:
        """The descriptor table for this cache: every entry's pools must lie in one group of full keys."""
        self.cache_id, self.table = id(cache), None
        groups = {cache.cache_group.get(e.cache) for e in self.model.spec.schedule}
        if len(groups) != 1:
            return
        gname = groups.pop()
        g = cache.kv_groups.get(gname)
        if g is None or g.request.window or g.k.dtype != torch.bfloat16:
            return
        dev = self.model.rt.device
        rows, maps = [], []
        keep = []
        for e, f in zip(self.model.spec.schedule, self.fields):
            m, ff = f["mixer"], f["ffn"]
            i = g.index[e.cache]
            k_pool, v_pool = g.k[i], g.v[i]
            inv = m["inv_freq"].to(device=dev, dtype=torch.float32).contiguous()
            keep += [inv, k_pool, v_pool]
            rows.append(struct.pack(
                "<9Q4i3fi", m["qkv"].data_ptr(), m["o"].data_ptr(), ff["gate_up"].data_ptr(), ff["down"].data_ptr(),
                f["mixer_norm"]["weight"].data_ptr(), f["ffn_norm"]["weight"].data_ptr(), k_pool.data_ptr(),
                v_pool.data_ptr(), inv.data_ptr(), m["num_heads"], m["num_kv_heads"], ff["intermediate_size"],
                ff["pair"], float(f["mixer_norm"]["eps"]), float(f["ffn_norm"]["eps"]),
                float(m["scale"]) * 1.4426950408889634, 0))
            maps += [K.decode_layers_encode_map(m["qkv"], self.hd // 2), K.decode_layers_encode_map(m["o"], 0),
                     K.decode_layers_encode_map(ff["gate_up"], ff["pair"]), K.decode_layers_encode_map(ff["down"], 0)]
        if self.head is not None:
            maps.append(K.decode_layers_encode_map(self.head["weight"], 0))
        blob = b"".join(rows)
        assert len(blob) == len(rows) * K.decode_layers_desc_bytes()
        self.keep = keep
        self.group = gname
        self.maps = torch.frombuffer(bytearray(b"".join(maps)), dtype=torch.uint8).to(dev)
        self.table = torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(dev)
        ctas, chunks = K.decode_layers_ctas(), K.decode_layers_max_chunks()
        bf = torch.bfloat16
        self.q = torch.empty(MAX_TOKENS, self.max_nh * self.hd, dtype=bf, device=dev)
        self.attn = torch.empty_like(self.q)
        self.act = torch.empty(MAX_TOKENS, self.max_I, dtype=bf, device=dev)
        self.xw = torch.empty(MAX_TOKENS, self.H, dtype=bf, device=dev)
        self.ssq = torch.zeros(2 * 16 * ((ctas + 3) // 4 * 4), dtype=torch.float32, device=dev)
        self.part_o = torch.empty(MAX_TOKENS * self.max_nh * chunks * self.hd, dtype=torch.float32, device=dev)
        self.part_ml = torch.empty(MAX_TOKENS * self.max_nh * chunks * 2, dtype=torch.float32, device=dev)
        self.sync = torch.zeros(4, dtype=torch.int32, device=dev)
        self.cand = torch.empty(MAX_TOKENS, ctas, 2, dtype=torch.float32, device=dev)
        self.x = torch.empty(MAX_TOKENS, self.H, dtype=torch.float32, device=dev)

    # ------------------------------------------------------------------ running
    def embeds(self) -> bool:
        """Whether ``run`` may be given no residual: the kernel then starts from the step's token ids."""
        return self.embedding is not None and self.with_head

    def run(self, h, step, cache, greedy: bool = False, note=None):
        """All layers on the residual stream ``h`` [T, H] (float32), in place (None: the kernel gathers the embedding
        rows itself; the residual is then ``self.last_h``). When the kernel can also take the final
        norm and the head and the step wants every token's result, it does, and the result comes back: the greedy
        tokens (int32 [T]; ``note`` as in ``LMHead.greedy``) or the logits (float32 [T, vocab]); else None."""
        self.runs += 1
        pt = step.page_tables[self.group]
        len_pages = (step.max_len + cache.page_size - 1) // cache.page_size
        result = None
        T = step.n_tokens
        if h is None:                                   # the kernel gathers the embedding rows into its own residual
            h = self.x[:T]
            K.decode_layers_set_embedding(self.embedding, step.tokens)
        self.last_h = h
        if self.head is not None and self.with_head and step.n_want == T:
            # every sequence brings one token and wants its result: the wanted rows are all rows, in order
            self.head_runs += 1
            hd = self.head
            if greedy:
                result = torch.empty(T, dtype=torch.int32, device=h.device)
                K.decode_layers_set_head(2, hd["weight"], hd["norm"], hd["eps"], self.cand, self.cand.shape[1])
                K.decode_layers_set_greedy_out(result, note)       # the kernel's last CTA takes the best candidates
            else:
                result = torch.empty(T, hd["vocab"], dtype=torch.float32, device=h.device)
                K.decode_layers_set_head(1, hd["weight"], hd["norm"], hd["eps"], result, hd["vocab"])
        K.decode_layers(self.table, self.maps, len(self.fields), step.n_tokens, self.H, self.hd, h, self.q, self.attn, self.act,
                        self.xw, self.ssq, self.part_o, self.part_ml, step.positions, step.seq_row, pt, cache.page_size,
                        len_pages, self.max_nkv, self.max_group, self.sync, plan=step.key_split,
                        n_pages=cache.kv_groups[self.group].n_pages)
        return result
