"""Short prompt steps with the host's work in C++: every layer's launch sequence in one call.

A prompt of a few dozen tokens is bound by the host, not the GPU: part by part a layer is eight launches of a few
microseconds each, and from Python each costs ten microseconds or more. When every layer's parts describe themselves
through ``fused_fields()`` (the description the one-kernel decode path and the fused prompt path read), a prompt step
of at most 128 tokens hands the whole sequence to ``csrc/host_step.cu``: a table of layer descriptors built once per
cache, the step's arrays and its activation buffers. Up to 16 tokens the kernels are the same as part by part, chosen
by the same thresholds (``parts/linear.py``), so the results are bit-identical to the Python path. From 17 to 64 tokens
(head sizes 64 and 128) a layer is five launches instead of eight: the norms, the rotation and the cache write ride in
the products' epilogues, the same kernels with the same arguments as ``engine/fused_prefill.py`` launches them, so
those results are bit-identical to that runner's. Anything else (another mixer, 32-bit, a larger step, a profiled
step) runs as before.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import torch

from ..csrc import lib as K
from ..parts import linear as L
from .fused_decode import collect_fused_fields

MAX_TOKENS = 128


class _Kernels(ctypes.Structure):
    _fields_ = [(n, c_void_p) for n in (
        "rmsnorm", "gemv", "gemv_supported", "tc_stream", "tc_stream_supported", "tc_gemm", "tc_gemm_supported",
        "gemm_generic", "silu_mul", "rope_kv_write", "flash_prefill", "err_generic", "err_gemv", "err_tc_stream",
        "err_tc_gemm", "err_attention", "tc_stream_fused", "rope_table", "norm_prepare")] + [("gemv_tokens", c_int), ("stream_tokens", c_int),
                                            ("flash_query_tile", c_int), ("pad", c_int)]


class _Layer(ctypes.Structure):
    _fields_ = [(n, c_void_p) for n in ("w_qkv", "w_o", "w_gu", "w_down", "norm1", "norm2", "k_pool", "v_pool", "inv_freq")] + \
               [(n, c_int) for n in ("nh", "nkv", "hd", "I", "gu_pair", "rotary_dim", "window", "pad")] + \
               [(n, c_float) for n in ("eps1", "eps2", "scale", "padf")]


class _Step(ctypes.Structure):
    _fields_ = [(n, c_void_p) for n in ("h", "x", "qkv", "q", "ctx", "act", "gu", "token_seq", "positions", "seq_row",
                                        "page_table", "seq_start", "status", "xw0", "xw1", "ssq0", "ssq1", "cs",
                                        "tok_page")] + \
               [(n, c_int) for n in ("T", "H", "n_seqs", "max_pages", "page_size", "n_q_tiles", "fused", "pad1")]


def _address(lib, name) -> int:
    return ctypes.cast(getattr(lib, name), c_void_p).value


_bound = False


def _bind() -> ctypes.CDLL:
    """Hand the other libraries' entry points to the C++ runner, once per process."""
    global _bound
    host = K.load("host_step")
    if _bound:
        return host
    for struct, size in ((_Kernels, "kernels"), (_Layer, "layer"), (_Step, "step")):
        want = int(getattr(host, f"sp_host_step_{size}_bytes")())
        if ctypes.sizeof(struct) != want:
            raise K.KernelError(f"host step: the {size} record has {ctypes.sizeof(struct)} bytes here, {want} in the library")
    generic, gemv, stream, gemm, att = (K.load(m) for m in ("generic", "gemv", "tc_stream", "tc_gemm", "attention"))
    t = _Kernels()
    t.rmsnorm, t.gemm_generic = _address(generic, "sp_rmsnorm"), _address(generic, "sp_gemm_generic")
    t.silu_mul, t.rope_kv_write = _address(generic, "sp_silu_mul"), _address(generic, "sp_rope_kv_write")
    t.gemv, t.gemv_supported = _address(gemv, "sp_gemv"), _address(gemv, "sp_gemv_supported")
    t.tc_stream, t.tc_stream_supported = _address(stream, "sp_tc_stream"), _address(stream, "sp_tc_stream_supported")
    t.tc_gemm, t.tc_gemm_supported = _address(gemm, "sp_tc_gemm"), _address(gemm, "sp_tc_gemm_supported")
    t.flash_prefill = _address(att, "sp_flash_prefill")
    t.tc_stream_fused = _address(stream, "sp_tc_stream_fused")
    t.rope_table, t.norm_prepare = _address(generic, "sp_rope_table"), _address(generic, "sp_norm_prepare")
    t.err_generic, t.err_gemv = _address(generic, "sp_generic_last_error"), _address(gemv, "sp_gemv_last_error")
    t.err_tc_stream, t.err_tc_gemm = _address(stream, "sp_tc_stream_last_error"), _address(gemm, "sp_tc_gemm_last_error")
    t.err_attention = _address(att, "sp_attention_last_error")
    t.gemv_tokens, t.stream_tokens = L.GEMV_TOKENS, L.STREAM_TOKENS
    t.flash_query_tile = K.flash_query_tile()
    K._check("host_step", host.sp_host_step_bind(ctypes.byref(t), ctypes.sizeof(t)))
    _bound = True
    return host


class HostStep:
    def __init__(self, model, fields: list):
        self.model = model
        self.fields = fields
        self.H = fields[0]["mixer"]["hidden_size"]
        self.runs = 0
        self.cache_id = None
        self.layers = None
        self.keep = None

    @classmethod
    def plan(cls, model):
        """A runner for ``model`` or None when some layer has to run part by part."""
        fields = collect_fused_fields(model)
        if fields is None:
            return None
        for f in fields:
            m = f["mixer"]
            hd = m["head_dim"]
            if hd % 16 or not 16 <= hd <= 128 or m["num_heads"] // m["num_kv_heads"] > 16:
                return None                              # the prompt attention kernel's sizes
        runner = cls(model, fields)
        from .fused_prefill import FusedPrefill
        runner.can_fuse = FusedPrefill.plan(model) is not None
        return runner

    def takes(self, step, cache) -> bool:
        if step.all_single or step.n_tokens > MAX_TOKENS or cache.page_size != K.flash_query_tile():
            return False
        if self.cache_id != id(cache):
            self._bind_cache(cache)
        return self.layers is not None

    def _bind_cache(self, cache) -> None:
        self.cache_id, self.layers = id(cache), None
        rows, keep, tables = [], [], []
        for e, f in zip(self.model.spec.schedule, self.fields):
            g = cache.kv_groups.get(cache.cache_group.get(e.cache))
            if g is None or g.request.window or g.k.dtype != torch.bfloat16:
                return
            m, ff = f["mixer"], f["ffn"]
            i = g.index[e.cache]
            k_pool, v_pool = g.k[i], g.v[i]
            inv = m["inv_freq"].to(device=k_pool.device, dtype=torch.float32).contiguous()
            for have in tables:                          # equal tables share one tensor: the runner compares addresses
                if have.shape == inv.shape and torch.equal(have, inv):
                    inv = have
                    break
            else:
                tables.append(inv)
            keep += [inv, k_pool, v_pool]
            r = _Layer()
            r.w_qkv, r.w_o, r.w_gu, r.w_down = (t.data_ptr() for t in (m["qkv"], m["o"], ff["gate_up"], ff["down"]))
            r.norm1, r.norm2 = f["mixer_norm"]["weight"].data_ptr(), f["ffn_norm"]["weight"].data_ptr()
            r.k_pool, r.v_pool, r.inv_freq = k_pool.data_ptr(), v_pool.data_ptr(), inv.data_ptr()
            r.nh, r.nkv, r.hd, r.I = m["num_heads"], m["num_kv_heads"], m["head_dim"], ff["intermediate_size"]
            r.gu_pair, r.rotary_dim, r.window = ff["pair"], m["head_dim"], 0
            r.eps1, r.eps2, r.scale = float(f["mixer_norm"]["eps"]), float(f["ffn_norm"]["eps"]), float(m["scale"])
            rows.append(r)
        self.keep = keep
        self.group = cache.cache_group[self.model.spec.schedule[0].cache]
        self.same_group = len({cache.cache_group.get(e.cache) for e in self.model.spec.schedule}) == 1
        if not self.same_group:
            return
        self.layers = (_Layer * len(rows))(*rows)
        self.max_qkv = max((r.nh + 2 * r.nkv) * r.hd for r in rows)
        self.max_q = max(r.nh * r.hd for r in rows)
        self.max_I = max(r.I for r in rows)

    def run(self, h: torch.Tensor, step, cache) -> None:
        """All layers on the residual stream ``h`` [T, H] (float32), in place."""
        host = _bind()
        self.runs += 1
        T, dev, bf = step.n_tokens, h.device, torch.bfloat16
        # one buffer for the step's activations (bfloat16 except the unrounded QKV products)
        n_bf = T * (self.H + 2 * self.max_q + self.max_I)
        work = torch.empty(n_bf * 2 + T * self.max_qkv * 4 + 64, dtype=torch.uint8, device=dev)
        base = work.data_ptr()
        base += (-base) % 16
        st = _Step()
        st.h = h.data_ptr()
        st.qkv = base
        off = base + T * self.max_qkv * 4
        st.x, off = off, off + T * self.H * 2
        st.q, off = off, off + T * self.max_q * 2
        st.ctx, off = off, off + T * self.max_q * 2
        st.act = off
        from .fused_prefill import fuses
        fused = self.can_fuse and self.model.fuse_prefill and fuses(T)
        if fused:
            tiles = K.tc_stream_n_tiles(self.H)
            hd = self.layers[0].hd
            extra = torch.empty(2 * T * self.H * 2 + 2 * T * tiles * 4 + T * hd * 4 + T * 4 + 64, dtype=torch.uint8, device=dev)
            off = extra.data_ptr()
            off += (-off) % 16
            st.xw0, off = off, off + T * self.H * 2
            st.xw1, off = off, off + T * self.H * 2
            st.ssq0, off = off, off + T * tiles * 4
            st.ssq1, off = off, off + T * tiles * 4
            st.cs, off = off, off + T * hd * 4                # (cos, sin) pairs of hd / 2 angles
            st.tok_page = off
            st.fused = 1
            self.extra = extra
        pt = step.page_tables[self.group]
        st.token_seq, st.positions, st.seq_row = step.token_seq.data_ptr(), step.positions.data_ptr(), step.seq_row.data_ptr()
        st.page_table, st.seq_start = pt.data_ptr(), step.seq_start.data_ptr()
        st.status = K.status_word(dev).data_ptr()
        st.T, st.H, st.n_seqs, st.max_pages, st.page_size = T, self.H, step.n_seqs, pt.shape[1], cache.page_size
        st.n_q_tiles = K.query_tiles(step.host["new_counts"], K.flash_query_tile())
        for module in ("generic", "attention", "gemv", "tc_gemm", "tc_stream"):       # the debug build's bounds, library by library
            K._declare_bounds(module, K.load(module), cache.kv_groups[self.group].n_pages, pt.shape[0], dev)
        stream = K._stream()
        rc = host.sp_host_step_prompt_layers(self.layers, len(self.fields), ctypes.byref(st), c_void_p(stream))
        K.launches += int(host.sp_host_step_launches()) - 1              # _stream() counted one
        K._check("host_step", rc)
        self.work = work                                                  # the allocator's stream order keeps it alive; so do we
