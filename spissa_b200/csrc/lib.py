"""ctypes bindings of the CUDA libraries: tensors in, a launch on the current stream.

Every function here launches a hand-written kernel; there is no CPU or library
fallback. A tensor that is not on a CUDA device, a library that cannot be built or a
size that a kernel refuses raises ``KernelError`` with the kernel's own words.
"""
from __future__ import annotations

import ctypes
from ctypes import c_void_p, c_int, c_float, c_longlong

import torch

from . import build

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


def dt_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 and bfloat16 tensors, got {t.dtype}") from None


_LIBS: dict = {}
_LOADED_PATHS: dict = {}


def load(module: str) -> ctypes.CDLL:
    """Build (if needed) and load one kernel library; cached per process."""
    lib = _LIBS.get(module)
    if lib is None:
        path = build.build_module(module)
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as e:
            raise KernelError(f"cannot load kernel library {path}: {e}") from None
        getattr(lib, f"sp_{module}_last_error").restype = ctypes.c_char_p
        _LIBS[module] = lib
        _LOADED_PATHS[module] = str(path)
        checked = getattr(lib, f"sp_{module}_range_checked", None)
        _RANGE_CHECKED[module] = bool(checked()) if checked is not None else False
    return lib


_RANGE_CHECKED: dict = {}


def range_checked(module: str) -> bool:
    """Whether ``module`` is loaded as the debug build whose kernels check table entries (see common.cuh)."""
    load(module)
    return _RANGE_CHECKED[module]


def _declare_bounds(module: str, lib, n_pages: int, n_rows: int, device) -> None:
    """Debug build only: the bounds the next launches of ``module`` check page and row indices against."""
    if _RANGE_CHECKED.get(module):
        getattr(lib, f"sp_{module}_set_bounds")(int(n_pages), int(n_rows), c_void_p(_ptr(status_word(device))))


def _table_rows(meta, pt) -> int:
    declared = getattr(meta, "declared_rows", None)
    return int(declared) if declared is not None else int(pt.shape[0])


def _pool_pages(meta, k_pool) -> int:
    """Pages of the pools; a harness may declare fewer than it allocated (``meta.declared_pages``) to see a check fire
    on an index that still lies inside allocated memory."""
    declared = getattr(meta, "declared_pages", None)
    return int(declared) if declared is not None else (int(k_pool.shape[0]) if k_pool is not None else 0)


def loaded_libraries() -> dict:
    return dict(_LOADED_PATHS)


def _check(module: str, rc: int) -> None:
    if rc != 0:
        msg = getattr(_LIBS[module], f"sp_{module}_last_error")()
        raise KernelError(msg.decode() if msg else f"kernel library {module} returned {rc}")


def _ptr(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernels run on CUDA tensors only; got a tensor on " + str(t.device))
    return t.data_ptr()


launches = 0          # kernels launched through these bindings since import (bench.py reports the difference)


# the current stream's handle without building a Stream object for every launch (a fifth of a launch's host time)
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    global launches
    launches += 1
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _need_contig(*ts):
    for t in ts:
        if t is not None and not t.is_contiguous():
            raise KernelError("kernels take contiguous tensors")


# ------------------------------------------------------------------ generic
def embed_gather(table, ids, out, status=None):
    """out[t,:] (float32) = table[ids[t],:]; an id outside the table zeroes the row and sets ``status``."""
    lib = load("generic")
    T, H = out.shape
    _need_contig(table, ids, out)
    _check("generic", lib.sp_embed_gather(
        c_void_p(_ptr(table)), dt_code(table), c_void_p(_ptr(ids)), c_void_p(_ptr(out)),
        T, H, table.shape[0], c_void_p(_ptr(status)), c_void_p(_stream())))


def rmsnorm(x, weight, out, eps, rows=None):
    """out[r,:] = x[rows[r] or r,:] / sqrt(mean(x²)+eps) · weight; ``x`` is float32."""
    lib = load("generic")
    if x.dtype != torch.float32:
        raise KernelError("rmsnorm reads the 32-bit residual stream")
    _need_contig(x, weight, out, rows)
    n_rows, H = out.shape
    _check("generic", lib.sp_rmsnorm(
        c_void_p(_ptr(x)), c_void_p(_ptr(weight)), dt_code(weight), c_void_p(_ptr(out)), dt_code(out),
        c_void_p(_ptr(rows)), n_rows, H, c_float(eps), c_void_p(_stream())))


def gemm_generic(a, w, out, accumulate=False):
    """out[M,N] (+)= a[M,K] · w[N,K]ᵀ with 32-bit FFMA accumulation, any sizes."""
    lib = load("generic")
    M, K = a.shape
    N, K2 = w.shape
    if K != K2 or out.shape[0] != M or out.shape[1] != N:
        raise KernelError(f"gemm shapes do not match: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm operands must have unit stride in their last dimension")
    _check("generic", lib.sp_gemm_generic(
        c_void_p(_ptr(a)), dt_code(a), c_void_p(_ptr(w)), dt_code(w), c_void_p(_ptr(out)), dt_code(out),
        M, N, K, a.stride(0), w.stride(0), out.stride(0), int(bool(accumulate)), c_void_p(_stream())))


def rope_kv_write(qkv, q_out, k_pool, v_pool, meta, inv_freq, nh, nkv, hd, rd, write_kv=True):
    """Rotate q and k of ``qkv`` [T, (nh+2·nkv)·hd], store q to ``q_out`` and k, v into the paged cache.

    ``meta`` carries ``token_seq``, ``positions``, ``seq_slot`` and the group's ``page_table``
    and ``page_size``. ``rd`` = 0 writes without rotating.
    """
    lib = load("generic")
    T = qkv.shape[0]
    _need_contig(qkv, q_out)
    pt = meta.page_table
    if pt is not None:
        _declare_bounds("generic", lib, _pool_pages(meta, k_pool), _table_rows(meta, pt), qkv.device)
    _check("generic", lib.sp_rope_kv_write(
        c_void_p(_ptr(qkv)), dt_code(qkv), c_void_p(_ptr(q_out)), dt_code(q_out),
        c_void_p(_ptr(k_pool)), c_void_p(_ptr(v_pool)), dt_code(k_pool) if k_pool is not None else 0,
        c_void_p(_ptr(meta.token_seq)), c_void_p(_ptr(meta.positions)), c_void_p(_ptr(meta.seq_slot)),
        c_void_p(_ptr(pt)), pt.shape[1] if pt is not None else 0, meta.page_size,
        c_void_p(_ptr(inv_freq)), T, nh, nkv, hd, rd, int(bool(write_kv)), c_void_p(_stream())))


def attention_generic(q, k_pool, v_pool, out, meta, nh, nkv, hd, window, scale):
    """Causal attention of every token of the step over its sequence's cached keys."""
    lib = load("generic")
    T = q.shape[0]
    _need_contig(q, out)
    pt = meta.page_table
    _declare_bounds("generic", lib, _pool_pages(meta, k_pool), _table_rows(meta, pt), q.device)
    _check("generic", lib.sp_attention_generic(
        c_void_p(_ptr(q)), dt_code(q), c_void_p(_ptr(k_pool)), c_void_p(_ptr(v_pool)), dt_code(k_pool),
        c_void_p(_ptr(out)), c_void_p(_ptr(meta.token_seq)), c_void_p(_ptr(meta.positions)),
        c_void_p(_ptr(meta.seq_slot)), c_void_p(_ptr(pt)), pt.shape[1], meta.page_size,
        T, nh, nkv, hd, int(window or 0), c_float(scale), c_void_p(_stream())))


def silu_mul(gu, out):
    """out[r,:] = silu(gu[r,:I]) ⊙ gu[r,I:]."""
    lib = load("generic")
    rows, I = out.shape
    _need_contig(gu, out)
    if gu.dtype != out.dtype or gu.shape[1] != 2 * I:
        raise KernelError("silu_mul wants gu [rows, 2·I] and out [rows, I] of one dtype")
    _check("generic", lib.sp_silu_mul(c_void_p(_ptr(gu)), c_void_p(_ptr(out)), dt_code(out), rows, I,
                                      c_void_p(_stream())))


def add_inplace(dst, src):
    """dst (float32) += src."""
    lib = load("generic")
    _need_contig(dst, src)
    if dst.dtype != torch.float32 or dst.numel() != src.numel():
        raise KernelError("add_inplace wants a float32 destination and equal sizes")
    _check("generic", lib.sp_add_inplace(c_void_p(_ptr(dst)), c_void_p(_ptr(src)), dt_code(src),
                                         c_longlong(dst.numel()), c_void_p(_stream())))


def gather_i32(src, idx, dst):
    """dst[i] = src[idx[i]] for int32 tensors on the device (indices outside ``src`` give 0)."""
    lib = load("generic")
    _need_contig(src, idx, dst)
    if src.dtype != torch.int32 or idx.dtype != torch.int32 or dst.dtype != torch.int32 or idx.numel() < dst.numel():
        raise KernelError("gather_i32 takes int32 tensors and one index per output")
    _check("generic", lib.sp_gather_i32(c_void_p(_ptr(src)), c_void_p(_ptr(idx)), c_void_p(_ptr(dst)), dst.numel(),
                                        src.numel(), c_void_p(_stream())))


def header_note(header, seq_slot, seq_len, tokens):
    """header[seq_slot[b]] = (seq_len[b], draws + 1, tokens[b], .) for every sequence b of a step."""
    lib = load("generic")
    _need_contig(header, seq_slot, seq_len, tokens)
    if any(t.dtype != torch.int32 for t in (header, seq_slot, seq_len, tokens)) or header.dim() != 2 or header.shape[1] != 4:
        raise KernelError("header_note takes int32 tensors and a header of four words per slot")
    n = tokens.numel()
    if seq_slot.numel() < n or seq_len.numel() < n:
        raise KernelError("header_note needs a slot and a length for every token")
    _check("generic", lib.sp_header_note(c_void_p(_ptr(header)), header.shape[0], c_void_p(_ptr(seq_slot)),
                                         c_void_p(_ptr(seq_len)), c_void_p(_ptr(tokens)), n, c_void_p(_stream())))


def wait_runs_out(device, code: int, limit_us: int, waited_ns=None):
    """Launch a kernel whose only wait, on a barrier nobody arrives on, gives up after ``limit_us`` microseconds and
    records ``code`` in the device's status word: how a bounded wait ends, for tests of the fault path."""
    lib = load("generic")
    _check("generic", lib.sp_wait_runs_out(c_void_p(_ptr(status_word(device))), int(code), c_longlong(int(limit_us)),
                                           c_void_p(_ptr(waited_ns)), c_void_p(_stream())))


def argmax_rows(logits, out):
    """out[r] = index of the first maximum of logits[r,:] (float32)."""
    lib = load("generic")
    rows, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("argmax wants float32 logits with unit column stride")
    _check("generic", lib.sp_argmax_rows(c_void_p(_ptr(logits)), c_void_p(_ptr(out)), rows, V,
                                         logits.stride(0), c_void_p(_stream())))


# ------------------------------------------------------------------ the greedy head: no logits
HEAD_ARGMAX_TOKENS = 64


def head_argmax_candidates(M: int, N: int) -> int:
    """Candidates per token that ``head_argmax`` needs room for (pairs of float32 and int32), 0 when it does not take M."""
    if M <= 16:
        return int(load("gemv").sp_gemv_argmax_candidates(int(N)))
    if M <= HEAD_ARGMAX_TOKENS:
        return int(load("tc_stream").sp_tc_stream_argmax_candidates(int(N)))
    return 0


def head_argmax_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    M = x.shape[0]
    if M <= 16:
        return gemv_supported(x, w)
    return M <= HEAD_ARGMAX_TOKENS and tc_stream_supported(x, w, 3)


def head_argmax(x, w, cand, out, note=None):
    """out[m] = argmax_n x[m]·w[n] (int32) without the logits: the product keeps one (value, row) candidate per tile
    of ``w`` and token in ``cand`` (float32 [M, head_argmax_candidates, 2] viewed as pairs), a second kernel takes the
    best of each row; the lowest row wins among equal values. ``note`` (an engine's ``step_note()``): the tokens also
    go into the headers of the step's sequences. Two kernels."""
    M, K = x.shape
    N = w.shape[0]
    n_cand = head_argmax_candidates(M, N)
    if n_cand == 0 or cand.dtype != torch.float32 or cand.numel() < M * n_cand * 2 or not cand.is_contiguous():
        raise KernelError(f"head_argmax: {M} tokens x {N} rows need a float32 table of {M}x{n_cand}x2")
    if out.dtype != torch.int32 or out.numel() < M:
        raise KernelError("head_argmax: the tokens go to an int32 tensor with one entry per row")
    if M <= 16:
        _check("gemv", load("gemv").sp_gemv_argmax(
            c_void_p(_ptr(x)), c_void_p(_ptr(w)), c_void_p(_ptr(cand)), M, N, K, x.stride(0), w.stride(0), n_cand,
            c_void_p(_stream())))
    else:
        _check("tc_stream", load("tc_stream").sp_tc_stream(
            c_void_p(_ptr(x)), c_void_p(_ptr(w)), c_void_p(_ptr(cand)), F32, M, N, K, x.stride(0), w.stride(0),
            n_cand, 3, 0, c_void_p(_ptr(status_word(x.device))), c_void_p(_stream())))
    header = note.header if note is not None else None
    _check("generic", load("generic").sp_argmax_candidates(
        c_void_p(_ptr(cand)), M, n_cand, n_cand, c_void_p(_ptr(out)), c_void_p(_ptr(header)),
        header.shape[0] if header is not None else 0,
        c_void_p(_ptr(note.seq_slot) if note is not None else None),
        c_void_p(_ptr(note.seq_len) if note is not None else None), c_void_p(_stream())))


# ------------------------------------------------------------------ sampling
def sample_scratch_keys(rows: int, V: int) -> int:
    lib = load("sampling")
    lib.sp_sample_scratch_keys.restype = c_longlong
    return int(lib.sp_sample_scratch_keys(rows, V))


def sample_rows(logits, temperature, top_k, top_p, u, scratch, out):
    """Temperature / top-k / top-p sampling of each row with the uniform numbers ``u``."""
    lib = load("sampling")
    rows, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sampling wants float32 logits with unit column stride")
    _check("sampling", lib.sp_sample_rows(
        c_void_p(_ptr(logits)), logits.stride(0), rows, V, c_float(temperature), int(top_k), c_float(top_p),
        c_void_p(_ptr(u)), c_void_p(_ptr(scratch)), c_longlong(scratch.numel()), c_void_p(_ptr(out)),
        c_void_p(_stream())))


# ------------------------------------------------------------------ tensor-core matrix product
_STATUS: dict = {}

STATUS_TEXT = {101: "the TMA loader waited too long for a free pipeline stage",
               102: "the MMA issuer waited too long for a loaded pipeline stage",
               103: "the epilogue waited too long for the accumulator",
               104: "the MMA issuer waited too long for a free accumulator",
               121: "tc_stream: the TMA loader waited too long for a free pipeline stage",
               122: "tc_stream: the MMA issuer waited too long for operands",
               123: "tc_stream: the epilogue warps waited too long for the accumulator",
               201: "decode layers: the copy warp waited too long for a free stage of the weight ring",
               202: "decode layers: a consumer warp waited too long for a weight tile",
               203: "decode layers: a CTA waited too long at the grid barrier",
               204: "decode layers: the split of the keys read from the device is outside what the scratch holds",
               205: "decode layers: a CTA waited too long for its partner's partial attention results",
               111: "attention: the loader waited too long for a free key/value stage",
               112: "attention: the MMA issuer waited too long for the queries",
               113: "attention: the MMA issuer waited too long for keys and values",
               114: "attention: the MMA issuer waited too long for the probabilities",
               115: "attention: the softmax warps waited too long for the scores",
               116: "attention: the softmax warps waited too long for the previous block's output",
               117: "attention: the softmax warps waited too long for the last block's output",
               301: "embedding: a token id outside the vocabulary",
               401: "range check: a page index from a page table lies beyond the pools",
               402: "range check: a sequence's row lies beyond the page table",
               403: "range check: a position lies beyond the page table's width",
               900: "a wait that was meant to run out (test of the fault path)"}


def status_word(device) -> torch.Tensor:
    """The int32 word in which kernels with bounded waits record that a wait ran out (0 = all well)."""
    key = torch.device(device).index or 0
    if key not in _STATUS:
        _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
    return _STATUS[key]


def check_status(device) -> None:
    """Synchronises and raises ``KernelError`` if a kernel gave up a wait since the last check."""
    key = torch.device(device).index or 0
    if key in _STATUS:
        code = int(_STATUS[key].item())
        if code:
            _STATUS[key].zero_()
            raise KernelError(f"a kernel gave up a bounded wait (code {code}: {STATUS_TEXT.get(code, 'unknown')})")


def tc_gemm_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``tc_gemm`` takes these operands (bfloat16, K-major, rows a multiple of 16 bytes)."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.dim() != 2 or w.dim() != 2:
        return False
    if a.stride(1) != 1 or w.stride(1) != 1 or a.shape[1] != w.shape[1]:
        return False
    K = a.shape[1]
    return (K % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


TC_STORE, TC_ACCUMULATE, TC_SILU_MUL = 0, 1, 2


def tc_gemm(a, w, out, mode=TC_STORE, bn=128):
    """out = a · wᵀ on the tcgen05 tensor cores (bfloat16 operands, float32 accumulation).

    ``mode`` TC_STORE writes ``out`` (bfloat16 or float32), TC_ACCUMULATE adds into a float32 ``out``,
    TC_SILU_MUL takes a weight whose rows interleave gate and up in blocks of ``bn``/2 and writes
    silu(gate)·up into ``out`` [M, N/2].
    """
    lib = load("tc_gemm")
    M, K = a.shape
    N = w.shape[0]
    want_cols = N // 2 if mode == TC_SILU_MUL else N
    if out.shape[0] != M or out.shape[1] != want_cols or out.stride(1) != 1:
        raise KernelError(f"tc_gemm: out {tuple(out.shape)} does not fit a {tuple(a.shape)}, w {tuple(w.shape)}")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("tc_gemm takes bfloat16 operands")
    _check("tc_gemm", lib.sp_tc_gemm(
        c_void_p(_ptr(a)), c_void_p(_ptr(w)), c_void_p(_ptr(out)), dt_code(out), M, N, K,
        a.stride(0), w.stride(0), out.stride(0), int(mode), int(bn), c_void_p(_ptr(status_word(a.device))),
        c_void_p(_stream())))


class _EpiArgs(ctypes.Structure):
    """Mirror of ``EpiArgs`` in tc_gemm.cu."""
    _fields_ = [("row_ssq", c_void_p), ("n_ssq", c_int), ("norm_width", c_int), ("eps", c_float), ("pad0", c_int),
                ("xw", c_void_p), ("next_w", c_void_p), ("ssq_out", c_void_p),
                ("cs", c_void_p), ("tok_page", c_void_p), ("positions", c_void_p),
                ("q_out", c_void_p), ("kpool", c_void_p), ("vpool", c_void_p),
                ("nh", c_int), ("nkv", c_int), ("hd", c_int), ("page_size", c_int)]


TC_QKV_ROPE = 3


def tc_gemm_splits(M: int, N: int, K: int, bn: int) -> int:
    """CTAs that share a tile along K when ``tc_gemm`` (the plain epilogues) runs these sizes; 1: K is not split."""
    return int(load("tc_gemm").sp_tc_gemm_splits(int(M), int(N), int(K), int(bn)))


def tc_gemm_n_tiles(N: int, bn: int) -> int:
    return (int(N) + int(bn) - 1) // int(bn)


def tc_gemm_fused(a, w, out, mode, bn, row_ssq=None, norm_width=0, eps=0.0, xw=None, next_w=None, ssq_out=None,
                  rope=None):
    """``tc_gemm`` with an epilogue that saves a pass over a prompt's activations.

    ``row_ssq`` [M, n] float32: ``a`` holds x ⊙ w of an RMS norm over ``norm_width`` columns without its 1/rms; the
    result is multiplied by 1/sqrt(sum(row_ssq[m]) / norm_width + eps).
    ``xw``, ``next_w``, ``ssq_out`` (mode TC_ACCUMULATE): besides out += a·wᵀ, xw = new out ⊙ next_w (bfloat16) and
    ssq_out[m, tile] = the new row's sum of squares over each tile's columns ([M, tc_gemm_n_tiles(N, bn)]).
    ``rope`` (mode TC_QKV_ROPE; ``out`` None): dict(cs, tok_page, positions, q_out, k_pool, v_pool, nh, nkv, hd,
    page_size): q and k are rotated with the (cos, sin) table, q stored, k and v written into the paged cache.
    """
    _fused_product("tc_gemm", a, w, out, mode, int(bn), tc_gemm_n_tiles(w.shape[0], bn), row_ssq, norm_width, eps, xw,
                   next_w, ssq_out, rope)


def tc_stream_max_tokens() -> int:
    """Tokens up to which ``tc_stream`` and ``tc_stream_fused`` are built."""
    return 128


def tc_stream_n_tiles(N: int) -> int:
    """Sums of squares per token that ``tc_stream_fused`` writes when it prepares the next norm (tiles of 128 columns)."""
    return (int(N) + 127) // 128


def tc_stream_fused(a, w, out, mode, pair=0, row_ssq=None, norm_width=0, eps=0.0, xw=None, next_w=None, ssq_out=None,
                    rope=None):
    """``tc_stream`` (17 to 128 tokens) with the epilogues of ``tc_gemm_fused``; ``ssq_out`` is
    [M, tc_stream_n_tiles(N)] here and ``pair`` the block of gate rows for TC_SILU_MUL."""
    _fused_product("tc_stream", a, w, out, mode, int(pair), tc_stream_n_tiles(w.shape[0]), row_ssq, norm_width, eps, xw,
                   next_w, ssq_out, rope)


def _fused_product(module, a, w, out, mode, width, n_tiles, row_ssq, norm_width, eps, xw, next_w, ssq_out, rope):
    lib = load(module)
    M, K = a.shape
    N = w.shape[0]
    ep = _EpiArgs()
    if row_ssq is not None:
        if row_ssq.dtype != torch.float32 or row_ssq.dim() != 2 or row_ssq.shape[0] < M or not row_ssq.is_contiguous():
            raise KernelError(f"{module}_fused: the row statistics are a contiguous float32 [M, n] tensor")
        ep.row_ssq, ep.n_ssq, ep.norm_width, ep.eps = _ptr(row_ssq), row_ssq.shape[1], int(norm_width), float(eps)
    if xw is not None:
        if (xw.dtype != torch.bfloat16 or tuple(xw.shape) != (M, N) or not xw.is_contiguous() or next_w.dtype != torch.bfloat16
                or next_w.numel() != N or ssq_out.dtype != torch.float32 or tuple(ssq_out.shape) != (M, n_tiles)
                or not ssq_out.is_contiguous()):
            raise KernelError(f"{module}_fused: xw [M, N] and next_w [N] are bfloat16, ssq_out float32 [M, {n_tiles}]")
        ep.xw, ep.next_w, ep.ssq_out = _ptr(xw), _ptr(next_w), _ptr(ssq_out)
    code = int(mode)
    if mode == TC_QKV_ROPE:
        r = rope
        _need_contig(r["cs"], r["tok_page"], r["positions"], r["q_out"])
        if r["q_out"].dtype != torch.bfloat16 or r["k_pool"].dtype != torch.bfloat16 or r["cs"].dtype != torch.float32:
            raise KernelError(f"{module}_fused: q and the cache are bfloat16, the angle table float32")
        ep.cs, ep.tok_page, ep.positions = _ptr(r["cs"]), _ptr(r["tok_page"]), _ptr(r["positions"])
        ep.q_out, ep.kpool, ep.vpool = _ptr(r["q_out"]), _ptr(r["k_pool"]), _ptr(r["v_pool"])
        ep.nh, ep.nkv, ep.hd, ep.page_size = int(r["nh"]), int(r["nkv"]), int(r["hd"]), int(r["page_size"])
        _declare_bounds(module, lib, r.get("declared_pages", r["k_pool"].shape[0]), 0, a.device)
        c_ptr, c_dt, ldc = None, BF16, 0
        if module == "tc_stream":
            code = 4                                   # 3 is the greedy head's mode there
    else:
        want_cols = N // 2 if mode == TC_SILU_MUL else N
        if out.shape[0] != M or out.shape[1] != want_cols or out.stride(1) != 1:
            raise KernelError(f"{module}_fused: out {tuple(out.shape)} does not fit a {tuple(a.shape)}, w {tuple(w.shape)}")
        c_ptr, c_dt, ldc = _ptr(out), dt_code(out), out.stride(0)
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"{module} takes bfloat16 operands")
    fn = lib.sp_tc_gemm_fused if module == "tc_gemm" else lib.sp_tc_stream_fused
    _check(module, fn(
        c_void_p(_ptr(a)), c_void_p(_ptr(w)), c_void_p(c_ptr), c_dt, M, N, K, a.stride(0), w.stride(0), ldc,
        code, width, ctypes.byref(ep), c_void_p(_ptr(status_word(a.device))), c_void_p(_stream())))


def rope_table(meta, inv_freq, half, cs, tok_page):
    """cs[t, i] = (cos, sin)(position[t] · inv_freq[i]) and tok_page[t] = the cache page of token t's position."""
    lib = load("generic")
    T = cs.shape[0]
    pt = meta.page_table
    _need_contig(cs, tok_page, inv_freq)
    _declare_bounds("generic", lib, _pool_pages(meta, getattr(meta, "k_pool", None)), _table_rows(meta, pt), cs.device)
    _check("generic", lib.sp_rope_table(
        c_void_p(_ptr(meta.positions)), c_void_p(_ptr(meta.token_seq)), c_void_p(_ptr(meta.seq_slot)),
        c_void_p(_ptr(pt)), pt.shape[1], meta.page_size, c_void_p(_ptr(inv_freq)), int(half), T, c_void_p(_ptr(cs)),
        c_void_p(_ptr(tok_page)), c_void_p(_stream())))


def norm_prepare(x, w, xw, ssq):
    """xw = x ⊙ w (bfloat16) and ssq[r] = sum of x[r]² for the float32 residual ``x`` [T, H]."""
    lib = load("generic")
    T, H = x.shape
    _need_contig(x, w, xw, ssq)
    if x.dtype != torch.float32 or w.dtype != torch.bfloat16 or xw.dtype != torch.bfloat16 or ssq.dtype != torch.float32:
        raise KernelError("norm_prepare: float32 residual and sums, bfloat16 weight and output")
    _check("generic", lib.sp_norm_prepare(c_void_p(_ptr(x)), c_void_p(_ptr(w)), c_void_p(_ptr(xw)), c_void_p(_ptr(ssq)),
                                          T, H, c_void_p(_stream())))


# ------------------------------------------------------------------ flash attention (bfloat16)
def flash_supported(q: torch.Tensor, k_pool: torch.Tensor, nh: int, nkv: int, hd: int, page_size: int) -> bool:
    """Whether the tensor-core attention kernels take this shape; else the generic kernel runs."""
    if q.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16:
        return False
    return bool(load("attention").sp_flash_supported(int(hd), int(nh), int(nkv), int(page_size)))


def flash_query_tile() -> int:
    """Query rows per CTA of ``flash_prefill``: a step has sum over sequences of ceil(new tokens / this) tiles."""
    return int(load("attention").sp_flash_query_tile())


def flash_tc_query_tile() -> int:
    """The same for ``flash_prefill_tc``."""
    return int(load("flash_tc").sp_flash_tc_query_tile())


def query_tiles(new_counts, tile: int) -> int:
    return sum((int(n) + tile - 1) // tile for n in new_counts)


def flash_prefill(q, k_pool, v_pool, out, meta, seq_start, n_seqs, n_q_tiles, nh, nkv, hd, window, scale):
    """Causal attention of a step's tokens (any number per sequence) over the paged cache.

    ``seq_start`` [B+1] int32 on the device; ``n_q_tiles`` = sum over sequences of ceil(new tokens /
    ``flash_query_tile()``).
    """
    lib = load("attention")
    _need_contig(q, out)
    pt = meta.page_table
    _declare_bounds("attention", lib, _pool_pages(meta, k_pool), _table_rows(meta, pt), q.device)
    _check("attention", lib.sp_flash_prefill(
        c_void_p(_ptr(q)), c_void_p(_ptr(out)), c_void_p(_ptr(k_pool)), c_void_p(_ptr(v_pool)),
        c_void_p(_ptr(seq_start)), c_void_p(_ptr(meta.positions)), c_void_p(_ptr(meta.seq_slot)),
        c_void_p(_ptr(pt)), pt.shape[1], meta.page_size, int(n_seqs), int(n_q_tiles), nh, nkv, hd,
        int(window or 0), c_float(scale), c_void_p(_stream())))


def flash_decode_plan(n_seqs: int, nkv: int, max_len: int, page_size: int = 64) -> tuple:
    """(tiles per chunk, chunks) for the split-key decode attention.

    Measured on B200 (head 64, 8 kv heads, 512 to 4096 keys): about 256 CTAs in all run fastest; with
    more than 256 (sequence, kv head) pairs two chunks beat one once there are 16 tiles or more.
    """
    tiles = max(1, (max_len + page_size - 1) // page_size)
    base = max(1, n_seqs * nkv)
    if base <= 256:
        n_chunks = min(8, max(1, round(256 / base)))
    else:
        n_chunks = 2 if tiles >= 16 else 1
    n_chunks = min(n_chunks, tiles)
    chunk_tiles = -(-tiles // n_chunks)
    n_chunks = -(-tiles // chunk_tiles)
    return chunk_tiles, n_chunks


def flash_decode_scratch_floats(n_seqs: int, nh: int, hd: int, n_chunks: int) -> int:
    return n_seqs * nh * n_chunks * (hd + 2)


def flash_decode(q, k_pool, v_pool, out, meta, seq_len, nh, nkv, hd, window, scale, chunk_tiles, n_chunks, scratch,
                 counters=None):
    """One query token per sequence: keys split into chunks over CTAs, partial results combined in order.

    ``seq_len`` [B] int32: each sequence's length including the query token. ``scratch``: float32,
    at least ``flash_decode_scratch_floats`` elements. ``counters``: int32, n_seqs·nkv zeros that the kernel
    hands back as zeros; with them the last CTA of each (sequence, kv head) combines, else a second kernel.
    """
    global launches
    lib = load("attention")
    _need_contig(q, out)
    pt = meta.page_table
    n_seqs = q.shape[0]
    if counters is not None and (counters.dtype != torch.int32 or counters.numel() < n_seqs * nkv):
        raise KernelError("flash_decode: counters must be int32 with a word per (sequence, kv head)")
    _declare_bounds("attention", lib, _pool_pages(meta, k_pool), _table_rows(meta, pt), q.device)
    _check("attention", lib.sp_flash_decode(
        c_void_p(_ptr(q)), c_void_p(_ptr(out)), dt_code(out), c_void_p(_ptr(k_pool)), c_void_p(_ptr(v_pool)),
        c_void_p(_ptr(seq_len)), c_void_p(_ptr(meta.seq_slot)), c_void_p(_ptr(pt)), pt.shape[1], meta.page_size,
        n_seqs, nh, nkv, hd, int(window or 0), c_float(scale), int(chunk_tiles), int(n_chunks),
        c_void_p(_ptr(scratch)), c_longlong(scratch.numel()), c_void_p(_ptr(counters)), c_void_p(_stream())))
    if counters is None:
        launches += 1        # two kernels: the chunks and the combine


# ------------------------------------------------------------------ skinny products for decoding
GEMV_MAX_TOKENS = 64


def gemv_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() != 2 or w.dim() != 2:
        return False
    if x.stride(1) != 1 or w.stride(1) != 1 or x.shape[1] != w.shape[1]:
        return False
    K = x.shape[1]
    return (0 < x.shape[0] <= GEMV_MAX_TOKENS and K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemv(x, w, out, mode=TC_STORE, pair=0):
    """out = x · wᵀ for up to 64 tokens, streaming ``w`` once. Modes as ``tc_gemm``; for TC_SILU_MUL
    ``pair`` is the number of gate rows before the matching up rows in the interleaved weight."""
    lib = load("gemv")
    M, K = x.shape
    N = w.shape[0]
    want_cols = N // 2 if mode == TC_SILU_MUL else N
    if out.shape[0] != M or out.shape[1] != want_cols or out.stride(1) != 1:
        raise KernelError(f"gemv: out {tuple(out.shape)} does not fit x {tuple(x.shape)}, w {tuple(w.shape)}")
    _check("gemv", lib.sp_gemv(
        c_void_p(_ptr(x)), c_void_p(_ptr(w)), c_void_p(_ptr(out)), dt_code(out), M, N, K,
        x.stride(0), w.stride(0), out.stride(0), int(mode), int(pair), c_void_p(_stream())))


def gemv_qkv_rope(x, w, q_out, k_pool, v_pool, meta, inv_freq, nh, nkv, hd):
    """The QKV product of a few tokens with rotate-half and the cache write in its epilogue.

    ``x`` bfloat16 [M, K]; ``w`` = [Wq; Wk; Wv]; q goes to ``q_out`` (bfloat16), k and v into the paged
    bfloat16 cache at each token's position.
    """
    lib = load("gemv")
    M, K = x.shape
    pt = meta.page_table
    if q_out.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemv_qkv_rope works on bfloat16 weights, queries and cache")
    _declare_bounds("gemv", lib, _pool_pages(meta, k_pool), _table_rows(meta, pt), x.device)
    _check("gemv", lib.sp_gemv_qkv_rope(
        c_void_p(_ptr(x)), x.stride(0), c_void_p(_ptr(w)), w.stride(0), M, K, nh, nkv, hd, c_void_p(_ptr(q_out)),
        c_void_p(_ptr(k_pool)), c_void_p(_ptr(v_pool)), c_void_p(_ptr(meta.positions)), c_void_p(_ptr(meta.token_seq)),
        c_void_p(_ptr(meta.seq_slot)), c_void_p(_ptr(pt)), pt.shape[1], meta.page_size, c_void_p(_ptr(inv_freq)),
        c_void_p(_stream())))


# ------------------------------------------------------------------ prefill attention on tcgen05
def flash_tc_supported(q: torch.Tensor, k_pool: torch.Tensor, nh: int, nkv: int, hd: int, page_size: int, window) -> bool:
    """Whether the tcgen05 prefill attention takes this shape (head 64 or 128, pages of 64, no window, bfloat16)."""
    return (q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and k_pool.is_contiguous()
            and bool(load("flash_tc").sp_flash_tc_supported(int(hd), int(nh), int(nkv), int(page_size), int(window or 0))))


def flash_prefill_tc(q, k_pool, v_pool, out, meta, seq_start, n_seqs, n_q_tiles, nh, nkv, hd, window, scale):
    """Causal attention of a step's tokens over the paged cache on the tcgen05 tensor cores.

    ``n_q_tiles`` = sum over sequences of ceil(new tokens / ``flash_tc_query_tile()``). S, P and O live in tensor memory.
    """
    lib = load("flash_tc")
    _need_contig(q, out, k_pool, v_pool)
    pt = meta.page_table
    _declare_bounds("flash_tc", lib, _pool_pages(meta, k_pool), _table_rows(meta, pt), q.device)
    _check("flash_tc", lib.sp_flash_prefill_tc(
        c_void_p(_ptr(q)), c_void_p(_ptr(out)), c_void_p(_ptr(k_pool)), c_void_p(_ptr(v_pool)),
        c_longlong(k_pool.shape[0]), q.shape[0], c_void_p(_ptr(seq_start)), c_void_p(_ptr(meta.positions)),
        c_void_p(_ptr(meta.seq_slot)), c_void_p(_ptr(pt)), pt.shape[1], meta.page_size, int(n_seqs), int(n_q_tiles),
        nh, nkv, hd, int(window or 0), c_float(scale), c_void_p(_ptr(status_word(q.device))), c_void_p(_stream())))


# ------------------------------------------------------------------ all layers of a decode step in one kernel
def decode_layers_ctas() -> int:
    return int(load("decode_layers").sp_decode_layers_ctas())


def decode_layers_max_chunks() -> int:
    return int(load("decode_layers").sp_decode_layers_max_chunks())


def decode_layers_max_pages() -> int:
    """Pages of the longest sequence that the kernel's split of the keys can hold."""
    return int(load("decode_layers").sp_decode_layers_max_pages())


def decode_layers_desc_bytes() -> int:
    return int(load("decode_layers").sp_decode_layers_desc_bytes())


def decode_layers_supported(T: int, H: int, hd: int, page_size: int, max_heads_per_kv: int) -> bool:
    return bool(load("decode_layers").sp_decode_layers_supported(int(T), int(H), int(hd), int(page_size),
                                                                 int(max_heads_per_kv)))


def decode_layers_encode_map(w: torch.Tensor, pair: int) -> bytes:
    """The TMA view of weight ``w`` [N, K] for the decode kernel's tile walk (rows in pairs ``pair`` apart; 0: plain)."""
    lib = load("decode_layers")
    _need_contig(w)
    n = int(lib.sp_decode_layers_map_bytes())
    buf = ctypes.create_string_buffer(n)
    _check("decode_layers", lib.sp_decode_layers_encode_map(buf, c_void_p(_ptr(w)), w.shape[0], w.shape[1], int(pair)))
    return buf.raw


def decode_layers(table, maps, n_layers, T, H, hd, x, q, attn, act, xw, ssq, part_o, part_ml, positions, seq_row, page_table,
                  page_size, len_pages, max_nkv, max_heads_per_kv, sync, plan=None, n_pages=0):
    """Every layer of a decode step (one token per sequence, T ≤ 16) on the residual ``x`` [T, H] float32, in place.

    ``table``: the layers' descriptors on the device (``decode_layers_desc_bytes()`` each). One cooperative launch;
    counts as one kernel. ``plan`` (two int32 on the device, from ``decode_layers_plan``) overrides the split of
    the keys that ``len_pages`` would give: a captured launch reads it anew at every replay.
    """
    lib = load("decode_layers")
    _need_contig(x, q, attn, act, page_table)
    if x.dtype != torch.float32 or x.shape[0] != T or x.shape[1] != H:
        raise KernelError(f"decode_layers: the residual must be float32 [{T}, {H}], got {x.dtype} {tuple(x.shape)}")
    _declare_bounds("decode_layers", lib, n_pages, page_table.shape[0], x.device)
    _check("decode_layers", lib.sp_decode_layers(
        c_void_p(_ptr(table)), c_void_p(_ptr(maps)), int(n_layers), int(T), int(H), int(hd), c_void_p(_ptr(x)), c_void_p(_ptr(q)),
        c_void_p(_ptr(attn)), c_void_p(_ptr(act)), c_void_p(_ptr(xw)), c_void_p(_ptr(ssq)), c_void_p(_ptr(part_o)), c_void_p(_ptr(part_ml)),
        c_void_p(_ptr(positions)), c_void_p(_ptr(seq_row)), c_void_p(_ptr(page_table)), page_table.shape[1],
        int(page_size), int(len_pages), int(max_nkv), int(max_heads_per_kv),
        c_void_p(_ptr(plan) if plan is not None else 0), c_void_p(_ptr(sync)),
        c_void_p(_ptr(status_word(x.device))), c_void_p(_stream())))


def decode_layers_set_head(mode: int, w, norm_w, eps: float, out, ld: int) -> None:
    """The output head of the NEXT ``decode_layers`` call: ``mode`` 1 writes logits [T, ld] (float32), 2 one (value,
    row) candidate per token and CTA [T, ld] (pairs of float32 and int32, for ``argmax_candidates``). The final norm
    (weight ``norm_w``, ``eps``) is folded into the product; the head's tensor map follows the layers' in ``maps``."""
    lib = load("decode_layers")
    _need_contig(w, norm_w, out)
    _check("decode_layers", lib.sp_decode_layers_set_head(
        int(mode), c_void_p(_ptr(w)), c_void_p(_ptr(norm_w)), c_float(eps), int(w.shape[0]), c_void_p(_ptr(out)), int(ld)))


def decode_layers_set_embedding(table, ids) -> None:
    """For the NEXT ``decode_layers`` call: the kernel fills the residual itself from the bfloat16 embedding ``table``
    [rows, H] and the token ``ids`` (int32 on the device); an id outside the table: a zero row and code 301."""
    lib = load("decode_layers")
    _need_contig(table, ids)
    if table.dtype != torch.bfloat16 or ids.dtype != torch.int32:
        raise KernelError("decode_layers: a bfloat16 embedding table and int32 token ids")
    _check("decode_layers", lib.sp_decode_layers_set_embedding(c_void_p(_ptr(table)), int(table.shape[0]), c_void_p(_ptr(ids))))


def decode_layers_set_greedy_out(tokens, note=None) -> None:
    """With head mode 2, for the NEXT ``decode_layers`` call: the kernel's last CTA also takes the best of each token's
    candidates and writes the tokens (int32 [T]); with ``note`` they also go into the headers of the step's sequences."""
    lib = load("decode_layers")
    header = note.header if note is not None else None
    _check("decode_layers", lib.sp_decode_layers_set_greedy_out(
        c_void_p(_ptr(tokens)), c_void_p(_ptr(header)), header.shape[0] if header is not None else 0,
        c_void_p(_ptr(note.seq_slot) if note is not None else None),
        c_void_p(_ptr(note.seq_len) if note is not None else None)))


def argmax_candidates(cand, rows: int, n_cand: int, out, note=None) -> None:
    """out[r] = the row of the best of ``cand[r, :n_cand]`` ((value, row) pairs; the lowest row among equal values);
    with ``note`` the tokens also go into the headers of the step's sequences."""
    header = note.header if note is not None else None
    _check("generic", load("generic").sp_argmax_candidates(
        c_void_p(_ptr(cand)), int(rows), int(n_cand), int(cand.shape[1]), c_void_p(_ptr(out)), c_void_p(_ptr(header)),
        header.shape[0] if header is not None else 0,
        c_void_p(_ptr(note.seq_slot) if note is not None else None),
        c_void_p(_ptr(note.seq_len) if note is not None else None), c_void_p(_stream())))


def decode_layers_plan(T: int, hd: int, len_pages: int, max_nkv: int) -> tuple:
    """(pages per chunk, chunks) of the keys for ``T`` sequences of at most ``len_pages`` pages."""
    lib = load("decode_layers")
    out = (ctypes.c_int * 2)()
    _check("decode_layers", lib.sp_decode_layers_plan(int(T), int(hd), int(len_pages), int(max_nkv), out))
    return int(out[0]), int(out[1])


# ------------------------------------------------------------------ weight-streaming tensor-core product (17..128 tokens)
def tc_stream_supported(x: torch.Tensor, w: torch.Tensor, mode=TC_STORE, pair: int = 0) -> bool:
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() != 2 or w.dim() != 2:
        return False
    if x.stride(1) != 1 or w.stride(1) != 1 or x.shape[1] != w.shape[1]:
        return False
    return load("tc_stream").sp_tc_stream_supported(
        c_void_p(_ptr(x)), c_void_p(_ptr(w)), x.shape[0], w.shape[0], x.shape[1], x.stride(0), w.stride(0),
        int(mode), int(pair)) == 0


def tc_stream(x, w, out, mode=TC_STORE, pair=0):
    """out = x · wᵀ for up to 128 tokens on the tensor cores with the rows of ``w`` as the instruction's M: every SM
    streams its share of ``w``; K is cut over the CTAs of a cluster, whose pieces are added in a fixed order. Modes as ``tc_gemm``; for
    TC_SILU_MUL ``pair`` is the number of gate rows before the matching up rows in the interleaved weight."""
    lib = load("tc_stream")
    M, K = x.shape
    N = w.shape[0]
    want_cols = N // 2 if mode == TC_SILU_MUL else N
    if out.shape[0] != M or out.shape[1] != want_cols or out.stride(1) != 1:
        raise KernelError(f"tc_stream: out {tuple(out.shape)} does not fit x {tuple(x.shape)}, w {tuple(w.shape)}")
    _check("tc_stream", lib.sp_tc_stream(
        c_void_p(_ptr(x)), c_void_p(_ptr(w)), c_void_p(_ptr(out)), dt_code(out), M, N, K, x.stride(0), w.stride(0),
        out.stride(0), int(mode), int(pair), c_void_p(_ptr(status_word(x.device))), c_void_p(_stream())))
