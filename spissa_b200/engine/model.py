"""A model put together from a ``ModelSpec``: embedding, layers in schedule order, norm, head.

The model class is the same for every architecture; what differs is the spec that the
architecture's configuration produces. Mirrors the reference's stateless forward
(crates/spissa-runtime/src/models/llama/api.rs:292-346): embedding, the blocks, the
final norm and the head — but only at the rows whose logits are wanted.
"""
from __future__ import annotations

import torch

from ..config.spec import ModelSpec
from ..parts import registry as part_registry
from ..parts.base import Runtime
from .. import parts as _parts  # noqa: F401  (registers the built-in parts)
from ..phases import phase, profiling


class Model:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.embedding = part_registry.build_part("embedding", spec.embedding)
        self.layers = []
        for layer in spec.layers:
            try:
                cls = part_registry._REGISTRY["block"][layer.block]
            except KeyError:
                raise ValueError(f"no block arrangement registered as {layer.block!r}; "
                                 f"known: {part_registry.known_parts('block')}") from None
            self.layers.append(cls(mixer=layer.mixer, ffn=layer.ffn, norms=layer.norms))
        self.final_norm = part_registry.build_part("norm", spec.final_norm)
        self.head = part_registry.build_part("head", spec.head)
        self.rt = None
        self.fuse_decode = True        # run a decode step's layers as one kernel when every layer's parts allow it
        self._fused = False            # False: not planned yet; None: the parts do not allow it
        self.fuse_prefill = True       # fold norms, rotation and cache write into a prompt step's products likewise
        self._fused_prefill = False
        self.host_steps = True         # a short prompt step's launch sequence as one call into C++ likewise
        self._host_step = False

    def kernel_modules(self, act_dtype) -> list:
        """The kernel libraries that steps of this model can need, for building them ahead of their first use (a guess
        costs processor time only: a library is still built when it is first asked for)."""
        if act_dtype != torch.bfloat16:
            return ["generic"]
        mods = ["generic", "gemv", "attention", "tc_gemm", "tc_stream"]
        head_sizes = {layer.mixer.params.get("head_dim") for layer in self.spec.layers}
        if head_sizes & {64, 128}:                  # the tcgen05 prompt attention, the one-kernel decode path, the C++ launcher
            mods += ["flash_tc", "decode_layers", "host_step"]
        return mods

    # ------------------------------------------------------------------ weights
    def parts(self) -> list:
        return [self.embedding] + self.layers + [self.final_norm, self.head]

    def weight_specs(self) -> list:
        out = []
        for p in self.parts():
            out.extend(p.all_weight_specs())
        return out

    def bind(self, tensors: dict, rt: Runtime) -> None:
        self.rt = rt
        for p in self.parts():
            p.bind_all(tensors, rt)

    def graph_safe(self) -> bool:
        """True when every part only launches kernels with device-side arguments (can be captured)."""
        def safe(p):
            return getattr(p, "graph_safe", False) and all(safe(c) for c in p.children())
        return all(safe(p) for p in self.parts())

    # ------------------------------------------------------------------ cache needs
    def cache_requests(self) -> dict:
        """cache id -> what the layer that writes it asks for."""
        out = {}
        for e in self.spec.schedule:
            if e.writes_cache:
                out[e.cache] = self.layers[e.layer].cache_request()
        return out

    def _host_runner(self, step, cache) -> bool:
        if self._host_step is False:
            from .host_step import HostStep
            self._host_step = HostStep.plan(self)
        return self._host_step is not None and self._host_step.takes(step, cache)

    # ------------------------------------------------------------------ forward
    def forward(self, step, cache, greedy: bool = False, note=None) -> torch.Tensor:
        """Logits [step.n_want, vocab] (float32) after running the step's tokens through every layer; with
        ``greedy`` the indices of their largest entries instead (int32 [step.n_want]; the logits are never written
        where the head has a kernel for that). ``note``: see ``LMHead.greedy``."""
        if self.fuse_decode and self._fused is False:
            from .fused_decode import FusedDecode
            self._fused = FusedDecode.plan(self)
        if self.fuse_prefill and self._fused_prefill is False:
            from .fused_prefill import FusedPrefill
            self._fused_prefill = FusedPrefill.plan(self)
        one_kernel = self.fuse_decode and self._fused is not None and not profiling() and self._fused.takes(step, cache)
        if one_kernel and self._fused.embeds():
            h = None                                       # the kernel gathers the embedding rows itself
        else:
            with phase("embedding_ms"):
                h = self.embedding.forward(step)
        if one_kernel:
            done = self._fused.run(h, step, cache, greedy, note)
            if done is not None:
                return done                                # the kernel ran the final norm and the head as well
            h = self._fused.last_h
        elif self.host_steps and not profiling() and self._host_runner(step, cache):
            self._host_step.run(h, step, cache)            # a prompt step of up to 128 tokens: launched from C++
        elif self.fuse_prefill and self._fused_prefill is not None and self._fused_prefill.takes(step, cache):
            self._fused_prefill.run(h, step, cache)
        else:
            for e in self.spec.schedule:
                self.layers[e.layer].forward(h, step, cache.view(e.cache, step, e.writes_cache))
        if step.n_want == 0:
            if greedy:
                return torch.empty(0, dtype=torch.int32, device=h.device)
            return torch.empty(0, self.spec.vocab_size, dtype=torch.float32, device=h.device)
        with phase("final_norm_ms"):
            x = self.final_norm.forward(h, rows=step.want_rows)
        if not greedy:
            with phase("lm_head_ms"):
                return self.head.forward(x)
        with phase("lm_head_ms"):
            tokens = self.head.greedy(x, note) if hasattr(self.head, "greedy") else None
        if tokens is None:
            # a head without such a kernel, or operands it does not take (32-bit, odd sizes): the logits, then their argmax
            from ..csrc import lib as K
            logits = self.head.forward(x)
            tokens = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
            K.argmax_rows(logits, tokens)
            if note is not None:
                K.header_note(note.header, note.seq_slot, note.seq_len, tokens)
        return tokens
