"""Run with SPISSA_B200_RANGE_CHECK=1 (tests/test_range_check_gpu.py does): the debug build's kernels report an index
that lies beyond the bounds the host DECLARED, and leave the access out. The pools and tables allocated here are
larger than what is declared, so every index used lies inside allocated memory whether or not a check fires: nothing
here relies on a check to stay inside memory."""
import math
import sys

import torch

import kernel_harness as KH
from spissa_b200.csrc import lib as K
from spissa_b200.csrc.lib import KernelError

DEV = "cuda:0"


def code_of(fn) -> int:
    """The status code that ``fn``'s launches leave (0: none)."""
    fn()
    try:
        K.check_status(DEV)
    except KernelError as e:
        text = str(e)
        return int(text.split("code ")[1].split(":")[0])
    return 0


def main() -> int:
    for module in ("generic", "attention", "gemv", "flash_tc", "tc_gemm", "decode_layers"):
        assert K.range_checked(module), f"{module} is not the debug build"
    torch.manual_seed(0)
    nh, nkv, hd = 8, 2, 64
    lengths = [200, 70]
    B = len(lengths)
    meta = KH.paged_meta([1] * B, [n - 1 for n in lengths], DEV, seed=3, spare_pages=4)
    ks = [torch.randn(n, nkv, hd) for n in lengths]
    vs = [torch.randn(n, nkv, hd) for n in lengths]
    k_pool, v_pool = KH.fill_cache(meta, ks, vs, nkv, hd, torch.bfloat16, DEV, junk=1.0)
    q = torch.randn(B, nh * hd, device=DEV).bfloat16()
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(hd)
    top_page = int(meta.page_table.max())

    def decode():
        ct, nc = K.flash_decode_plan(B, nkv, max(lengths))
        scratch = torch.empty(K.flash_decode_scratch_floats(B, nh, hd, nc), device=DEV)
        K.flash_decode(q, k_pool, v_pool, out, meta, meta.seq_len, nh, nkv, hd, None, scale, ct, nc, scratch)

    assert code_of(decode) == 0                                   # true bounds: nothing to report
    meta.declared_pages = top_page                                # the highest page in the table now lies beyond the bound
    assert code_of(decode) == 401
    meta.declared_pages = None
    meta.declared_rows = 1                                        # the second sequence's row lies beyond the bound
    assert code_of(decode) == 402
    meta.declared_rows = None

    def generic_attention():
        K.attention_generic(q, k_pool, v_pool, out, meta, nh, nkv, hd, None, scale)
    assert code_of(generic_attention) == 0
    meta.declared_pages = top_page
    assert code_of(generic_attention) == 401
    meta.declared_pages = None

    # the cache write of a prompt step: a token whose page lies beyond the declared pools is reported and NOT written
    new_counts, before = [40, 9], [0, 100]
    wmeta = KH.paged_meta(new_counts, before, DEV, seed=5, spare_pages=4)
    T = sum(new_counts)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV)
    inv_freq = torch.ones(hd // 2, device=DEV) * 0.01
    qo = torch.empty(T, nh * hd, dtype=torch.bfloat16, device=DEV)

    def write(declared):
        kp = torch.full((wmeta.n_pages, nkv, 64, hd), 9.0, dtype=torch.bfloat16, device=DEV)
        vp = torch.full_like(kp, -9.0)
        wmeta.declared_pages = declared
        code = code_of(lambda: K.rope_kv_write(qkv, qo, kp, vp, wmeta, inv_freq, nh, nkv, hd, hd))
        wmeta.declared_pages = None
        return code, kp
    code, kp = write(None)
    assert code == 0 and bool((kp[wmeta.rows[0][0]] != 9.0).any())
    bad = max(wmeta.rows[0] + wmeta.rows[1])
    code, kp = write(bad)
    assert code == 401 and bool((kp[bad] == 9.0).all())           # that page was left alone
    other = [p for p in wmeta.rows[0] + wmeta.rows[1] if p != bad]
    assert any(bool((kp[p] != 9.0).any()) for p in other)          # the tokens of the other pages were written

    # the same through the tensor-core QKV epilogue of a fused prompt step
    H = 128
    xw = torch.randn(T, H, device=DEV).bfloat16()
    w = (torch.randn((nh + 2 * nkv) * hd, H, device=DEV) * 0.1).bfloat16()
    cs = torch.empty(T, hd // 2, 2, device=DEV)
    tok_page = torch.empty(T, dtype=torch.int32, device=DEV)
    K.rope_table(wmeta, inv_freq, hd // 2, cs, tok_page)
    K.check_status(DEV)

    def fused(declared):
        kp = torch.full((wmeta.n_pages, nkv, 64, hd), 9.0, dtype=torch.bfloat16, device=DEV)
        vp = torch.full_like(kp, -9.0)
        rope = dict(cs=cs, tok_page=tok_page, positions=wmeta.positions, q_out=qo, k_pool=kp, v_pool=vp, nh=nh, nkv=nkv,
                    hd=hd, page_size=64)
        if declared is not None:
            rope["declared_pages"] = declared
        return code_of(lambda: K.tc_gemm_fused(xw, w, None, K.TC_QKV_ROPE, 128, rope=rope)), kp
    code, kp = fused(None)
    assert code == 0
    code, kp = fused(bad)
    assert code == 401 and bool((kp[bad] == 9.0).all())

    # and through the same epilogue of the kernel that streams the weights (steps of 17 to 64 tokens)
    assert K.range_checked("tc_stream")

    def streamed(declared):
        kp = torch.full((wmeta.n_pages, nkv, 64, hd), 9.0, dtype=torch.bfloat16, device=DEV)
        vp = torch.full_like(kp, -9.0)
        rope = dict(cs=cs, tok_page=tok_page, positions=wmeta.positions, q_out=qo, k_pool=kp, v_pool=vp, nh=nh, nkv=nkv,
                    hd=hd, page_size=64)
        if declared is not None:
            rope["declared_pages"] = declared
        return code_of(lambda: K.tc_stream_fused(xw, w, None, K.TC_QKV_ROPE, 0, rope=rope)), kp
    code, kp = streamed(None)
    assert code == 0
    code, kp = streamed(bad)
    assert code == 401 and bool((kp[bad] == 9.0).all())
    assert any(bool((kp[p] != 9.0).any()) for p in other)
    print("range check cases ok")
    return 0


if __name__ == "__main__":
    sys.exit(main())
