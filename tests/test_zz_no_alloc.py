"""The decode-attention entry point that brings its own scratch (csrc/attention_noalloc.h).

Some programs that embed the kernels cannot allocate device memory when they need attention (a
server whose pool owns all of the GPU's memory, a host that forbids allocation after start-up), so
``sp_flash_decode_static`` keeps its scratch in an array inside the library. This test calls it
through its exported C symbol, twice in a row with different inputs, and compares each result with
the regular entry point, which takes the scratch from its caller. The file name sorts last so that a
run that stops at the first failure has already run every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

import kernel_harness as KH

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def one_case(K, lib, seed, lengths, nh, nkv, hd, chunk_tiles, out_dtype=torch.bfloat16, window=None):
    torch.manual_seed(seed)
    B = len(lengths)
    meta = KH.paged_meta([1] * B, [n - 1 for n in lengths], DEV, seed)
    ks = [torch.randn(n, nkv, hd).bfloat16().float() for n in lengths]
    vs = [torch.randn(n, nkv, hd).bfloat16().float() for n in lengths]
    k_pool, v_pool = KH.fill_cache(meta, ks, vs, nkv, hd, torch.bfloat16, DEV)
    q = torch.randn(B, nh * hd, device=DEV).bfloat16()
    scale = 1.0 / math.sqrt(hd)
    n_chunks = -(-((max(lengths) + 63) // 64) // chunk_tiles)

    want = torch.empty(q.shape, dtype=out_dtype, device=DEV)
    scratch = torch.empty(K.flash_decode_scratch_floats(B, nh, hd, n_chunks), device=DEV)
    counters = torch.zeros(B * nkv, dtype=torch.int32, device=DEV)
    K.flash_decode(q, k_pool, v_pool, want, meta, meta.seq_len, nh, nkv, hd, window, scale, chunk_tiles, n_chunks,
                   scratch, counters)

    got = torch.full_like(want, float("nan"))
    rc = lib.sp_flash_decode_static(
        c_void_p(q.data_ptr()), c_void_p(got.data_ptr()), 1 if out_dtype == torch.bfloat16 else 0,
        c_void_p(k_pool.data_ptr()), c_void_p(v_pool.data_ptr()),
        c_void_p(meta.seq_len.data_ptr()), c_void_p(meta.seq_slot.data_ptr()), c_void_p(meta.page_table.data_ptr()),
        meta.page_table.shape[1], 64, B, nh, nkv, hd, int(window or 0), c_float(scale), chunk_tiles, n_chunks,
        c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.sp_attention_last_error().decode()
    torch.cuda.synchronize()
    ref = KH.plain_attention_rows([torch.cat([torch.zeros(n - 1, nh, hd), q[b].float().cpu().reshape(1, nh, hd)])
                                   for b, n in enumerate(lengths)], ks, vs, [1] * B, window=window)
    scale_ref = float(ref.abs().max())
    # the same kernel, the same split of the keys, the chunks combined in the same order: not a bit may differ
    assert torch.equal(got, want)
    assert float((got.double().cpu() - ref.reshape(B, -1)).abs().max()) <= 6e-3 * scale_ref


def test_static_scratch_entry_point_matches_the_regular_one_twice_in_a_row():
    from spissa_b200.csrc import lib as K
    lib = K.load("attention")
    lib.sp_attention_last_error.restype = ctypes.c_char_p
    torch.cuda.set_device(0)
    one_case(K, lib, 1, [700, 64, 129, 300], 8, 2, 64, 2)
    one_case(K, lib, 2, [33, 1000], 4, 1, 128, 3)


def test_static_scratch_entry_point_with_float32_output_and_with_a_window():
    from spissa_b200.csrc import lib as K
    lib = K.load("attention")
    lib.sp_attention_last_error.restype = ctypes.c_char_p
    torch.cuda.set_device(0)
    one_case(K, lib, 3, [500, 90], 8, 2, 64, 2, out_dtype=torch.float32)
    one_case(K, lib, 4, [700, 64, 300], 4, 2, 64, 3, window=100)
    one_case(K, lib, 5, [260, 131], 20, 2, 128, 2, out_dtype=torch.float32, window=70)      # ten query heads per kv head


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from spissa_b200.csrc import lib as K
    lib = K.load("attention")
    lib.sp_attention_last_error.restype = ctypes.c_char_p
    dummy = torch.zeros(16, device=DEV)
    p = c_void_p(dummy.data_ptr())
    # 64 sequences x 32 heads x 64 chunks x 66 floats is far beyond the 2^20 floats of the built-in array
    rc = lib.sp_flash_decode_static(p, p, 1, p, p, p, p, p, 64, 64, 64, 32, 8, 64, 0, c_float(0.125), 1, 64,
                                    c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 1
    assert "built-in array holds" in lib.sp_attention_last_error().decode()
