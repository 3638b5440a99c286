"""Each kernel alone against its plain reference, at sizes other than the engine's tiny models."""
import math
import random

import pytest
import torch

import kernel_harness as KH
from plain import llama_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def K():
    from spissa_b200.csrc import lib
    return lib


def close(got, ref, tol, what=""):
    err = float((got.double().cpu() - ref.double().cpu()).abs().max())
    scale = float(ref.double().abs().max()) or 1.0
    assert err <= tol * scale, f"{what}: error {err:.3e} against scale {scale:.3e} (allowed {tol:.1e} of it)"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_gather(K, dtype):
    torch.manual_seed(0)
    V, H = 333, 72
    table = torch.randn(V, H).to(dtype)
    ids = torch.tensor([0, 332, 17, 17, 200], dtype=torch.int32)
    out = torch.empty(5, H, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.embed_gather(table.to(DEV), ids.to(DEV), out, status)
    assert torch.equal(out.cpu(), P.embedding(table.float(), ids.tolist()))
    assert int(status.item()) == 0
    bad = torch.tensor([1, 333], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, H, dtype=torch.float32, device=DEV)
    K.embed_gather(table.to(DEV), bad, out2, status)
    assert int(status.item()) == 301 and float(out2[1].abs().max()) == 0.0     # code 301: an id outside the table


@pytest.mark.parametrize("H", [72, 512, 1000, 2048, 3072, 4096, 4100])
@pytest.mark.parametrize("wdt,odt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.float32, torch.bfloat16)])
def test_rmsnorm(K, H, wdt, odt):
    torch.manual_seed(1)
    x = torch.randn(9, H) * 3
    w = (1 + 0.1 * torch.randn(H)).to(wdt)
    rows = torch.tensor([8, 0, 3, 3], dtype=torch.int32)
    ref = P.rms_norm(x.double(), w.double(), 1e-6)
    out = torch.empty(9, H, dtype=odt, device=DEV)
    K.rmsnorm(x.to(DEV), w.to(DEV), out, 1e-6)
    close(out, ref, 2e-6 if odt == torch.float32 else 4e-3, "all rows")
    out = torch.empty(4, H, dtype=odt, device=DEV)
    K.rmsnorm(x.to(DEV), w.to(DEV), out, 1e-6, rows.to(DEV))
    close(out, ref[rows.long()], 2e-6 if odt == torch.float32 else 4e-3, "gathered rows")


@pytest.mark.parametrize("M,N,K_", [(1, 7, 5), (33, 130, 72), (100, 64, 200), (5, 333, 96), (64, 64, 16),
                                    (1, 130, 72), (16, 1030, 520), (8, 100, 2048), (3, 7, 4), (2, 9, 1028), (17, 40, 512)])
@pytest.mark.parametrize("adt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.bfloat16, torch.float32), (torch.float32, torch.bfloat16)])
def test_gemm_generic(K, M, N, K_, adt, wdt):
    torch.manual_seed(2)
    a = torch.randn(M, K_).to(adt)
    w = torch.randn(N, K_).to(wdt)
    ref = a.double() @ w.double().t()
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    K.gemm_generic(a.to(DEV), w.to(DEV), out)
    close(out, ref, 2e-6, "float32 out")
    base = torch.randn(M, N)
    acc = base.clone().to(DEV)
    K.gemm_generic(a.to(DEV), w.to(DEV), acc, accumulate=True)
    close(acc, ref + base.double(), 2e-6, "accumulate")
    outb = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    K.gemm_generic(a.to(DEV), w.to(DEV), outb)
    close(outb, ref, 4e-3, "bfloat16 out")


def test_gemm_row_does_not_depend_on_batch(K):
    """A row's result is the same bit for bit whatever else is in the batch, within the kernel for a few rows (a
    decode step: up to 16) and within the tiled kernel; between the two it differs by 32-bit rounding only."""
    torch.manual_seed(3)
    a = torch.randn(70, 200, device=DEV)
    w = torch.randn(90, 200, device=DEV)
    full = torch.empty(70, 90, device=DEV)
    K.gemm_generic(a, w, full)
    some = torch.empty(20, 90, device=DEV)
    K.gemm_generic(a[30:50].contiguous(), w, some)
    assert torch.equal(some[7], full[37])
    one = torch.empty(1, 90, device=DEV)
    K.gemm_generic(a[37:38].contiguous(), w, one)
    for rows in (2, 3, 8, 11, 16):
        few = torch.empty(rows, 90, device=DEV)
        K.gemm_generic(a[37:37 + rows].contiguous(), w, few)
        assert torch.equal(few[0], one[0]), rows
    close(one[0], full[37].double().cpu(), 2e-6, "a few rows against the tiled kernel")


def rope_case(K, nh, nkv, hd, rd, theta, dtype, new_counts, before, seed):
    torch.manual_seed(seed)
    T = sum(new_counts)
    meta = KH.paged_meta(new_counts, before, DEV, seed)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd)
    inv = P.rope_inv_freq(theta, rd) if rd else None
    q_out = torch.empty(T, nh * hd, dtype=dtype, device=DEV)
    k_pool = torch.zeros(meta.n_pages, nkv, KH.PAGE, hd, dtype=dtype, device=DEV)
    v_pool = torch.zeros_like(k_pool)
    K.rope_kv_write(qkv.to(DEV), q_out, k_pool, v_pool, meta, inv.to(DEV) if rd else None, nh, nkv, hd, rd)
    pos = meta.positions.cpu()
    q = qkv[:, :nh * hd].reshape(T, nh, hd)
    k = qkv[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd)
    v = qkv[:, (nh + nkv) * hd:].reshape(T, nkv, hd)
    if rd:
        q, k = P.apply_rope(q, pos, inv), P.apply_rope(k, pos, inv)
    tol = 2e-6 if dtype == torch.float32 else 4e-3
    close(q_out, q.reshape(T, -1), tol, "q")
    seq = meta.token_seq.cpu()
    for t in range(T):
        b, p = int(seq[t]), int(pos[t])
        pg, off = meta.rows[b][p // KH.PAGE], p % KH.PAGE
        close(k_pool[pg, :, off, :], k[t], tol, f"k of token {t}")
        close(v_pool[pg, :, off, :], v[t], tol, f"v of token {t}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,rd", [(4, 2, 16, 16), (3, 1, 32, 32), (3, 3, 48, 24), (8, 2, 128, 128),
                                          (2, 2, 64, 0)])
def test_rope_kv_write(K, dtype, nh, nkv, hd, rd):
    rope_case(K, nh, nkv, hd, rd, 10000.0, dtype, [5, 1, 70], [0, 130, 60], seed=nh * 100 + hd)


def attention_case(K, fn, nh, nkv, hd, dtype, new_counts, before, window, seed, tol):
    torch.manual_seed(seed)
    B = len(new_counts)
    meta = KH.paged_meta(new_counts, before, DEV, seed)
    qs = [torch.randn(t, nh, hd) for t in meta.total_len]
    ks = [torch.randn(t, nkv, hd) for t in meta.total_len]
    vs = [torch.randn(t, nkv, hd) for t in meta.total_len]
    if dtype == torch.bfloat16:
        qs, ks, vs = ([x.bfloat16().float() for x in xs] for xs in (qs, ks, vs))
    k_pool, v_pool = KH.fill_cache(meta, ks, vs, nkv, hd, dtype, DEV)
    q = torch.cat([qb[-n:] for qb, n in zip(qs, new_counts)], 0).reshape(-1, nh * hd).to(dtype).to(DEV)
    out = torch.empty_like(q)
    fn(q, k_pool, v_pool, out, meta, nh, nkv, hd, window, 1.0 / math.sqrt(hd))
    ref = KH.plain_attention_rows(qs, ks, vs, new_counts, window)
    close(out, ref, tol, f"attention nh={nh} nkv={nkv} hd={hd} window={window}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (3, 1, 32), (3, 3, 48), (8, 2, 64), (4, 1, 128), (2, 1, 256)])
def test_attention_generic_prefill_and_decode(K, dtype, nh, nkv, hd):
    tol = 3e-6 if dtype == torch.float32 else 6e-3
    attention_case(K, K.attention_generic, nh, nkv, hd, dtype, [7, 1, 65, 33], [0, 199, 64, 31], None, hd, tol)
    attention_case(K, K.attention_generic, nh, nkv, hd, dtype, [1, 1, 1], [0, 63, 300], None, hd + 1, tol)


@pytest.mark.parametrize("window", [1, 5, 64, 100])
def test_attention_generic_window(K, window):
    attention_case(K, K.attention_generic, 4, 2, 32, torch.float32, [40, 1, 130], [0, 250, 20], window, window, 3e-6)


def needle_case(K, fn, dtype, length, needle, window=None, hd=64, nh=4, nkv=2):
    """One key among ``length`` scores far above the rest: the output must be that key's value."""
    torch.manual_seed(length + needle)
    meta = KH.paged_meta([1], [length - 1], DEV, seed=needle)
    k = torch.randn(length, nkv, hd) * 0.1
    v = torch.randn(length, nkv, hd)
    q = torch.randn(1, nh, hd) * 0.1
    k[needle] = 0
    k[needle, :, 0] = 40.0
    q[0, :, 0] = 40.0
    if dtype == torch.bfloat16:
        q, k, v = q.bfloat16().float(), k.bfloat16().float(), v.bfloat16().float()
    k_pool, v_pool = KH.fill_cache(meta, [k], [v], nkv, hd, dtype, DEV)
    qd = q.reshape(1, nh * hd).to(dtype).to(DEV)
    out = torch.empty_like(qd)
    fn(qd, k_pool, v_pool, out, meta, nh, nkv, hd, window, 1.0 / math.sqrt(hd))
    return out.float().cpu().reshape(nh, hd), v


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("length,needle", [(700, 3), (700, 640), (129, 64), (64, 63), (1000, 0)])
def test_attention_generic_finds_a_far_key(K, dtype, length, needle):
    out, v = needle_case(K, K.attention_generic, dtype, length, needle)
    for h in range(4):
        assert torch.allclose(out[h], v[needle, h // 2], atol=2e-2), f"head {h} missed key {needle} of {length}"


def test_attention_generic_window_edge(K):
    # the key at p-window+1 is seen, the key at p-window is not
    length, window = 300, 100
    p = length - 1
    out, v = needle_case(K, K.attention_generic, torch.float32, length, p - window + 1, window)
    assert torch.allclose(out[0], v[p - window + 1, 0], atol=2e-2)
    out, v = needle_case(K, K.attention_generic, torch.float32, length, p - window, window)
    assert not torch.allclose(out[0], v[p - window, 0], atol=0.5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul(K, dtype):
    torch.manual_seed(4)
    gu = (torch.randn(7, 2 * 136) * 3).to(dtype)
    out = torch.empty(7, 136, dtype=dtype, device=DEV)
    K.silu_mul(gu.to(DEV), out)
    ref = P.silu(gu[:, :136].double()) * gu[:, 136:].double()
    close(out, ref, 2e-6 if dtype == torch.float32 else 4e-3)


def test_add_inplace(K):
    torch.manual_seed(5)
    a, b = torch.randn(1000), torch.randn(1000).bfloat16()
    d = a.clone().to(DEV)
    K.add_inplace(d, b.to(DEV))
    assert torch.equal(d.cpu(), a + b.float())


def test_argmax_first_maximum_wins(K):
    torch.manual_seed(6)
    logits = torch.randn(5, 128256)
    logits[1, 777] = logits[1, 90000] = 50.0
    logits[2, :] = 0.0
    logits[3, 128255] = 60.0
    logits[4, 5] = float("nan")
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    K.argmax_rows(logits.to(DEV), out)
    want = [P.sample_argmax(logits[0].tolist()), 777, 0, 128255, P.sample_argmax(logits[4].tolist())]
    assert out.tolist() == want


def walk64(logits_row, temp, k, p, u):
    """The reference's walk in float64: (ordering, running mass, kept count, target)."""
    probs = torch.softmax(logits_row.double() / temp, 0)
    order = sorted(range(len(probs)), key=lambda i: (-float(probs[i]), i))
    kept = min(k, len(order)) if k > 0 else len(order)
    cum = torch.cumsum(probs[order[:kept]], 0)
    reach = (cum >= p).nonzero()
    if len(reach):
        kept = int(reach[0]) + 1
    edge = float(probs[order[kept - 1]])            # the top-p cut compares a rounded sum: one token either way
    return order, cum, kept, u * float(cum[kept - 1]), edge


@pytest.mark.parametrize("V", [7, 333, 4096, 5000, 128256])
def test_sampling_follows_the_reference_walk(K, V):
    torch.manual_seed(V)
    rows = 6
    logits = torch.randn(rows, V) * 2.5
    logits[0, :] = 0.0                                         # all equal: order by index
    cases = [(0.8, 0, 0.95), (1.0, 1, 1.0), (1.3, 5, 0.5), (0.7, 0, 1.0), (1.0, 50, 0.9)]
    scratch = torch.empty(K.sample_scratch_keys(rows, V), dtype=torch.int64, device=DEV)
    for temp, k, p in cases:
        for seed in ((1, 2, 3) if V <= 6000 else (1,)):
            us = [P.seeded_unit_f32(seed * 100 + r) for r in range(rows)]
            out = torch.empty(rows, dtype=torch.int32, device=DEV)
            K.sample_rows(logits.to(DEV), temp, k, p, torch.tensor(us, device=DEV), scratch, out)
            got = out.tolist()
            for r in range(rows if V <= 6000 else 3):
                # in float64 the chosen token's stretch of the running mass holds the draw, up to the
                # rounding of 32-bit sums (1e-5 of the kept mass)
                order, cum, kept, target, edge = walk64(logits[r], temp, k, p, us[r])
                rank = order.index(got[r])
                assert rank <= kept, (V, temp, k, p, r, "outside the kept set")
                lo = float(cum[rank - 1]) if rank > 0 else 0.0
                hi = float(cum[min(rank, kept - 1)])
                slack = 1e-5 * float(cum[kept - 1]) + (edge if p < 1.0 else 0.0)
                assert lo - slack <= target <= hi + slack, (V, temp, k, p, r, got[r], lo, target, hi)
                if V <= 5000 and r > 0:
                    # and it is the serial 32-bit walk's choice or its neighbour
                    want = P.sample_top_k_top_p(logits[r].tolist(), temp, k, p, seed * 100 + r)
                    assert abs(rank - order.index(want)) <= 1, (V, temp, k, p, r, got[r], want)


def test_sampling_row_too_long_for_shared_memory(K):
    """Above 262,144 tokens a slice of the row no longer fits the shared memory and the passes read the
    probabilities from the scratch row; above 524,287 the kernel refuses."""
    V, rows = 270001, 2
    torch.manual_seed(5)
    logits = torch.randn(rows, V) * 4
    scratch = torch.empty(K.sample_scratch_keys(rows, V), dtype=torch.int64, device=DEV)
    for temp, k, p in [(0.9, 0, 0.9), (1.0, 30, 1.0)]:
        us = [P.seeded_unit_f32(17 + r) for r in range(rows)]
        out = torch.empty(rows, dtype=torch.int32, device=DEV)
        K.sample_rows(logits.to(DEV), temp, k, p, torch.tensor(us, device=DEV), scratch, out)
        for r in range(rows):
            order, cum, kept, target, edge = walk64(logits[r], temp, k, p, us[r])
            rank = order.index(int(out[r]))
            assert rank <= kept
            lo = float(cum[rank - 1]) if rank > 0 else 0.0
            hi = float(cum[min(rank, kept - 1)])
            slack = 1e-5 * float(cum[kept - 1]) + (edge if p < 1.0 else 0.0)
            assert lo - slack <= target <= hi + slack, (temp, k, p, r, int(out[r]), lo, target, hi)
    big = torch.zeros(1, 600000, device=DEV)
    with pytest.raises(Exception, match="beyond this kernel"):
        K.sample_rows(big, 1.0, 0, 1.0, torch.zeros(1, device=DEV), torch.empty(300000, dtype=torch.int64, device=DEV),
                      torch.empty(1, dtype=torch.int32, device=DEV))


def test_sampling_ties_and_repeats(K):
    """Groups of exactly equal probabilities are walked by rising index, and the same draw gives the same token
    every time (the sums are integers: no order of addition can change them)."""
    V, rows = 128256, 4
    torch.manual_seed(11)
    logits = torch.randn(rows, V)
    logits[0, :] = -10.0
    logits[0, 1000:1016] = 10.0                                # 16 equal tokens hold all the mass but 2e-5
    logits[1] = torch.round(logits[1] * 2) / 2                 # thousands of ties everywhere
    logits[2, 77] = 40.0                                       # one token holds all of it
    scratch = torch.empty(K.sample_scratch_keys(rows, V), dtype=torch.int64, device=DEV)
    dev_logits = logits.to(DEV)
    for temp, k, p in [(1.0, 0, 0.9), (0.5, 8, 1.0), (1.0, 0, 1.0)]:
        firsts = None
        for seed in range(6):
            us = [P.seeded_unit_f32(seed * 31 + r) for r in range(rows)]
            u = torch.tensor(us, device=DEV)
            out = torch.empty(rows, dtype=torch.int32, device=DEV)
            K.sample_rows(dev_logits, temp, k, p, u, scratch, out)
            got = out.tolist()
            for _ in range(3):
                again = torch.empty(rows, dtype=torch.int32, device=DEV)
                K.sample_rows(dev_logits, temp, k, p, u, scratch, again)
                assert again.tolist() == got
            assert got[2] == 77
            # row 0: the draw falls into the 16 equal tokens, the u-th of them by index (their mass is ~1)
            probs = torch.softmax(logits[0].double() / temp, 0)
            each, rest = float(probs[1000]), float(probs[0])
            kept = 16 if (k == 0 or k >= 16) else k
            if p < 1.0 and p <= kept * each:
                kept = min(kept, int(-(-p // each)))
            if k == 0 and p == 1.0:
                want_rank = int(us[0] * 1.0 / each) if us[0] < 16 * each else None
            else:
                want_rank = min(kept - 1, int(us[0] * kept))
            if want_rank is not None and abs(us[0] * kept - round(us[0] * kept)) > 1e-3:
                assert got[0] == 1000 + want_rank, (temp, k, p, seed, got[0], want_rank)
            for r in (1, 3):
                order, cum, kept_r, target, edge = walk64(logits[r], temp, k, p, us[r])
                rank = order.index(got[r])
                assert rank <= kept_r
                lo = float(cum[rank - 1]) if rank > 0 else 0.0
                hi = float(cum[min(rank, kept_r - 1)])
                slack = 1e-5 * float(cum[kept_r - 1]) + (edge if p < 1.0 else 0.0)
                assert lo - slack <= target <= hi + slack, (temp, k, p, seed, r, got[r], lo, target, hi)


# ------------------------------------------------------------------ tensor-core attention (bfloat16)
def flash_prefill_fn(K):
    def fn(q, k_pool, v_pool, out, meta, nh, nkv, hd, window, scale):
        n_tiles = sum((c + 63) // 64 for c in meta.new_counts)
        K.flash_prefill(q, k_pool, v_pool, out, meta, meta.seq_start, len(meta.new_counts), n_tiles, nh, nkv, hd,
                        window, scale)
    return fn


def flash_decode_fn(K, chunk_tiles=None, fused=True):
    counters = torch.zeros(1024, dtype=torch.int32, device=DEV) if fused else None

    def fn(q, k_pool, v_pool, out, meta, nh, nkv, hd, window, scale):
        ct, nc = K.flash_decode_plan(q.shape[0], nkv, max(meta.total_len))
        if chunk_tiles:
            ct = chunk_tiles
            nc = -(-((max(meta.total_len) + 63) // 64) // ct)
        scratch = torch.full((K.flash_decode_scratch_floats(q.shape[0], nh, hd, nc),), float("nan"), device=DEV)
        K.flash_decode(q, k_pool, v_pool, out, meta, meta.seq_len, nh, nkv, hd, window, scale, ct, nc, scratch,
                       counters)
        if fused:
            assert int(counters.abs().sum()) == 0          # handed back at zero for the next launch
    return fn


@pytest.mark.parametrize("nh,nkv,hd", [(8, 2, 64), (4, 4, 64), (3, 1, 64), (4, 1, 128), (16, 1, 128), (6, 3, 128),
                                       (4, 2, 16), (3, 1, 32), (3, 3, 48), (6, 2, 80), (5, 1, 96), (4, 2, 112)])
def test_flash_prefill(K, nh, nkv, hd):
    fn = flash_prefill_fn(K)
    attention_case(K, fn, nh, nkv, hd, torch.bfloat16, [7, 1, 65, 33], [0, 199, 64, 31], None, hd, 6e-3)
    attention_case(K, fn, nh, nkv, hd, torch.bfloat16, [300, 64, 128], [0, 0, 100], None, hd + 2, 6e-3)
    attention_case(K, fn, nh, nkv, hd, torch.bfloat16, [1, 1, 1], [0, 63, 300], None, hd + 1, 6e-3)


@pytest.mark.parametrize("window", [1, 5, 64, 100, 200])
def test_flash_prefill_window(K, window):
    attention_case(K, flash_prefill_fn(K), 4, 2, 64, torch.bfloat16, [40, 1, 230], [0, 250, 20], window, window, 6e-3)


@pytest.mark.parametrize("nh,nkv,hd", [(8, 2, 64), (4, 4, 64), (3, 1, 64), (4, 1, 128), (16, 1, 128), (32, 8, 64), (10, 1, 64),
                                       (16, 2, 64), (9, 1, 128), (4, 2, 16), (3, 1, 32), (3, 3, 48), (6, 2, 80), (10, 1, 96),
                                       (4, 2, 112)])
@pytest.mark.parametrize("chunk_tiles", [None, 1, 3])
@pytest.mark.parametrize("fused", [True, False])
def test_flash_decode(K, nh, nkv, hd, chunk_tiles, fused):
    fn = flash_decode_fn(K, chunk_tiles, fused)
    attention_case(K, fn, nh, nkv, hd, torch.bfloat16, [1, 1, 1, 1, 1], [0, 63, 64, 300, 700], None, hd + 3, 6e-3)


@pytest.mark.parametrize("window", [1, 5, 64, 100, 200])
def test_flash_decode_window(K, window):
    attention_case(K, flash_decode_fn(K, 2), 4, 2, 64, torch.bfloat16, [1, 1, 1], [0, 250, 20], window, window, 6e-3)


@pytest.mark.parametrize("which", ["prefill", "decode"])
@pytest.mark.parametrize("length,needle", [(700, 3), (700, 640), (129, 64), (64, 63), (1000, 0), (65, 64)])
def test_flash_finds_a_far_key(K, which, length, needle):
    fn = flash_prefill_fn(K) if which == "prefill" else flash_decode_fn(K)
    out, v = needle_case(K, fn, torch.bfloat16, length, needle)
    for h in range(4):
        assert torch.allclose(out[h], v[needle, h // 2], atol=2e-2), f"head {h} missed key {needle} of {length}"


@pytest.mark.parametrize("which", ["prefill", "decode"])
@pytest.mark.parametrize("hd", [16, 48, 96, 112])
def test_flash_finds_a_far_key_at_other_head_sizes(K, which, hd):
    fn = flash_prefill_fn(K) if which == "prefill" else flash_decode_fn(K)
    out, v = needle_case(K, fn, torch.bfloat16, 700, 640, hd=hd)
    for h in range(4):
        assert torch.allclose(out[h], v[640, h // 2], atol=2e-2), f"head {h} of size {hd} missed key 640 of 700"


@pytest.mark.parametrize("which", ["prefill", "decode"])
def test_flash_window_edge(K, which):
    fn = flash_prefill_fn(K) if which == "prefill" else flash_decode_fn(K)
    length, window = 300, 100
    p = length - 1
    out, v = needle_case(K, fn, torch.bfloat16, length, p - window + 1, window)
    assert torch.allclose(out[0], v[p - window + 1, 0], atol=2e-2)
    out, v = needle_case(K, fn, torch.bfloat16, length, p - window, window)
    assert not torch.allclose(out[0], v[p - window, 0], atol=0.5)


def test_flash_ignores_junk_beyond_the_sequence(K):
    """Rows of the last page beyond the sequence's end hold huge values; no query may see them."""
    for fn, counts, before in ((flash_prefill_fn(K), [70], [0]), (flash_decode_fn(K), [1], [69])):
        attention_case(K, fn, 4, 2, 64, torch.bfloat16, counts, before, None, 5, 6e-3)


# ------------------------------------------------------------------ tensor-core products (bfloat16)
def interleave(gate, up, h):
    I = gate.shape[0]
    return torch.stack([gate.reshape(I // h, h, -1), up.reshape(I // h, h, -1)], dim=1).reshape(2 * I, -1).contiguous()


@pytest.mark.parametrize("M,N,K_", [(1, 8, 8), (1, 333, 72), (8, 3072, 2048), (3, 100, 200), (16, 2048, 8192),
                                    (17, 72, 96), (32, 520, 264), (64, 2048, 2048), (33, 7, 40)])
def test_gemv(K, M, N, K_):
    torch.manual_seed(M * 1000 + N)
    x = torch.randn(M, K_).bfloat16()
    w = torch.randn(N, K_).bfloat16()
    ref = x.double() @ w.double().t()
    for odt, tol in ((torch.float32, 3e-6), (torch.bfloat16, 4e-3)):
        out = torch.full((M, N), 9.0, dtype=odt, device=DEV)
        K.gemv(x.to(DEV), w.to(DEV), out)
        close(out, ref, tol, f"store {odt}")
    base = torch.randn(M, N)
    acc = base.clone().to(DEV)
    K.gemv(x.to(DEV), w.to(DEV), acc, mode=K.TC_ACCUMULATE)
    close(acc, ref + base.double(), 3e-6, "accumulate")


@pytest.mark.parametrize("M,I,K_,h", [(1, 64, 72, 64), (8, 8192, 2048, 128), (5, 192, 64, 64), (20, 256, 96, 128),
                                      (64, 384, 200, 64)])
def test_gemv_silu_mul(K, M, I, K_, h):
    torch.manual_seed(I + M)
    x = torch.randn(M, K_).bfloat16()
    g, u = (torch.randn(I, K_) * 0.2).bfloat16(), (torch.randn(I, K_) * 0.2).bfloat16()
    ref = P.silu(x.double() @ g.double().t()) * (x.double() @ u.double().t())
    out = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    K.gemv(x.to(DEV), interleave(g, u, h).to(DEV), out, mode=K.TC_SILU_MUL, pair=h)
    close(out, ref, 4e-3)


def test_gemv_is_repeatable_and_row_independent(K):
    torch.manual_seed(9)
    x = torch.randn(8, 2048, device=DEV).bfloat16()
    w = torch.randn(512, 2048, device=DEV).bfloat16()
    a = torch.empty(8, 512, device=DEV)
    b = torch.empty(8, 512, device=DEV)
    K.gemv(x, w, a)
    K.gemv(x, w, b)
    assert torch.equal(a, b)
    one = torch.empty(1, 512, device=DEV)
    K.gemv(x[5:6].contiguous(), w, one)
    assert torch.equal(one[0], a[5])


@pytest.mark.parametrize("M,N,K_,bn", [(128, 128, 64, 128), (100, 72, 96, 128), (1, 333, 72, 128), (300, 200, 200, 128),
                                       (257, 520, 136, 256), (2048, 3072, 2048, 256), (129, 256, 8, 256),
                                       # one row of tiles and a long K: the cluster splits K
                                       (64, 3072, 2048, 128), (17, 2048, 8192, 128), (128, 200, 1000, 128),
                                       (100, 130, 520, 256), (33, 2048, 2048, 256),
                                       # 192-wide tiles: whole, ragged in M and N, many tiles per CTA, one row of tiles
                                       (2048, 3072, 2048, 192), (300, 200, 136, 192), (129, 5120, 72, 192), (64, 3072, 2048, 192),
                                       # from 1,024 rows on pairs of CTAs compute tiles of 256 rows (cta_group::2): ragged in M
                                       # and N, a last tile whose second CTA has no rows, more tiles than pairs
                                       (1024, 256, 64, 128), (1025, 520, 136, 128), (1500, 1160, 264, 192), (1300, 300, 72, 256),
                                       (1152, 20480, 128, 256), (4096, 2048, 512, 256),
                                       # several rows of few tiles and a long K: the cluster splits K there too
                                       (256, 2048, 8192, 128), (300, 520, 4100 - 4, 256), (129, 200, 4096, 128), (511, 1030, 4160, 128)])
def test_tc_gemm(K, M, N, K_, bn):
    torch.manual_seed(M + N)
    a = torch.randn(M, K_).bfloat16()
    w = torch.randn(N, K_).bfloat16()
    ref = a.double() @ w.double().t()
    for odt, tol in ((torch.float32, 3e-6), (torch.bfloat16, 4e-3)):
        out = torch.full((M, N), 9.0, dtype=odt, device=DEV)
        K.tc_gemm(a.to(DEV), w.to(DEV), out, bn=bn)
        close(out, ref, tol, f"store {odt}")
    base = torch.randn(M, N)
    acc = base.clone().to(DEV)
    K.tc_gemm(a.to(DEV), w.to(DEV), acc, mode=K.TC_ACCUMULATE, bn=bn)
    close(acc, ref + base.double(), 3e-6, "accumulate")
    K.check_status(DEV)


@pytest.mark.parametrize("M,I,K_,bn", [(200, 256, 96, 128), (130, 1024, 72, 256), (64, 192, 64, 128),
                                       (64, 1024, 2048, 256), (20, 8192, 2048, 256), (128, 256, 1000, 128)])
def test_tc_gemm_silu_mul(K, M, I, K_, bn):
    torch.manual_seed(I)
    a = torch.randn(M, K_).bfloat16()
    g, u = (torch.randn(I, K_) * 0.2).bfloat16(), (torch.randn(I, K_) * 0.2).bfloat16()
    ref = P.silu(a.double() @ g.double().t()) * (a.double() @ u.double().t())
    out = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    K.tc_gemm(a.to(DEV), interleave(g, u, bn // 2).to(DEV), out, mode=K.TC_SILU_MUL, bn=bn)
    close(out, ref, 4e-3)
    K.check_status(DEV)


# ------------------------------------------------------------------ the tensor-core product that streams W (up to 128 tokens)
@pytest.mark.parametrize("M,N,K_", [(17, 3072, 2048), (64, 2048, 8192), (1, 130, 72), (33, 200, 1000), (128, 520, 136),
                                     (100, 128, 64), (48, 2048, 2048), (16, 136, 8), (65, 1000, 520)])
def test_tc_stream(K, M, N, K_):
    torch.manual_seed(M + N)
    a = torch.randn(M, K_).bfloat16()
    w = torch.randn(N, K_).bfloat16()
    ref = a.double() @ w.double().t()
    assert K.tc_stream_supported(a.to(DEV), w.to(DEV))
    for odt, tol in ((torch.float32, 3e-6), (torch.bfloat16, 4e-3)):
        out = torch.full((M, N), 9.0, dtype=odt, device=DEV)
        K.tc_stream(a.to(DEV), w.to(DEV), out)
        close(out, ref, tol, f"store {odt}")
    base = torch.randn(M, N)
    acc = base.clone().to(DEV)
    K.tc_stream(a.to(DEV), w.to(DEV), acc, mode=K.TC_ACCUMULATE)
    close(acc, ref + base.double(), 3e-6, "accumulate")
    again = base.clone().to(DEV)
    K.tc_stream(a.to(DEV), w.to(DEV), again, mode=K.TC_ACCUMULATE)
    assert torch.equal(acc, again), "the pieces of K are added in a fixed order: two runs agree bit for bit"
    K.check_status(DEV)


@pytest.mark.parametrize("M,I,K_,block", [(20, 8192, 2048, 128), (64, 1024, 2048, 128), (64, 192, 64, 64), (33, 256, 1000, 128),
                                           (128, 256, 72, 128), (17, 320, 208, 64), (5, 128, 136, 128)])
def test_tc_stream_silu_mul(K, M, I, K_, block):
    torch.manual_seed(I)
    a = torch.randn(M, K_).bfloat16()
    g, u = (torch.randn(I, K_) * 0.2).bfloat16(), (torch.randn(I, K_) * 0.2).bfloat16()
    ref = P.silu(a.double() @ g.double().t()) * (a.double() @ u.double().t())
    out = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    w = interleave(g, u, block).to(DEV)
    assert K.tc_stream_supported(a.to(DEV), w, K.TC_SILU_MUL, block)
    K.tc_stream(a.to(DEV), w, out, mode=K.TC_SILU_MUL, pair=block)
    close(out, ref, 4e-3)
    K.check_status(DEV)


def test_tc_stream_refuses_what_it_cannot_do(K):
    a = torch.randn(4, 12, device=DEV).bfloat16()
    w = torch.randn(4, 12, device=DEV).bfloat16()
    assert not K.tc_stream_supported(a, w)                                        # rows of 24 bytes
    big = torch.randn(129, 64, device=DEV).bfloat16()
    assert not K.tc_stream_supported(big, torch.randn(8, 64, device=DEV).bfloat16())     # more than 128 tokens
    with pytest.raises(K.KernelError, match="1 to 128 tokens"):
        K.tc_stream(big, torch.randn(8, 64, device=DEV).bfloat16(), torch.empty(129, 8, device=DEV))


def test_tc_gemm_refuses_rows_that_tma_cannot_fetch(K):
    a = torch.randn(4, 12, device=DEV).bfloat16()
    w = torch.randn(4, 12, device=DEV).bfloat16()
    assert not K.tc_gemm_supported(a, w) and not K.gemv_supported(a, w)
    with pytest.raises(K.KernelError, match="multiples of 8"):
        K.tc_gemm(a, w, torch.empty(4, 4, device=DEV))
    with pytest.raises(K.KernelError, match="multiples of 8"):
        K.gemv(a, w, torch.empty(4, 4, device=DEV))


# ------------------------------------------------------------------ the decode QKV product with rotation and cache write
@pytest.mark.parametrize("nh,nkv,hd,H", [(4, 2, 16, 64), (3, 1, 32, 96), (8, 2, 64, 256), (4, 1, 128, 200), (3, 3, 48, 72)])
def test_gemv_qkv_rope(K, nh, nkv, hd, H):
    torch.manual_seed(nh * 10 + hd)
    new_counts, before = [1, 3, 1, 2], [0, 130, 63, 64]
    T = sum(new_counts)
    meta = KH.paged_meta(new_counts, before, DEV, seed=hd)
    x = torch.randn(T, H).bfloat16()
    w = (torch.randn((nh + 2 * nkv) * hd, H) * 0.2).bfloat16()
    inv = P.rope_inv_freq(10000.0, hd)
    q_out = torch.zeros(T, nh * hd, dtype=torch.bfloat16, device=DEV)
    k_pool = torch.zeros(meta.n_pages, nkv, KH.PAGE, hd, dtype=torch.bfloat16, device=DEV)
    v_pool = torch.zeros_like(k_pool)
    K.gemv_qkv_rope(x.to(DEV), w.to(DEV), q_out, k_pool, v_pool, meta, inv.to(DEV), nh, nkv, hd)
    qkv = (x.double() @ w.double().t()).float()
    pos = meta.positions.cpu()
    q = P.apply_rope(qkv[:, :nh * hd].reshape(T, nh, hd), pos, inv)
    k = P.apply_rope(qkv[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd), pos, inv)
    v = qkv[:, (nh + nkv) * hd:].reshape(T, nkv, hd)
    close(q_out, q.reshape(T, -1), 4e-3, "q")
    seq = meta.token_seq.cpu()
    for t in range(T):
        b, p = int(seq[t]), int(pos[t])
        pg, off = meta.rows[b][p // KH.PAGE], p % KH.PAGE
        close(k_pool[pg, :, off, :], k[t], 4e-3, f"k of token {t}")
        close(v_pool[pg, :, off, :], v[t], 4e-3, f"v of token {t}")


@pytest.mark.parametrize("M,N,K_", [(1, 19000, 72), (8, 20008, 264), (16, 19004, 96)])
def test_gemv_many_rows_streams_without_splitting_k(K, M, N, K_):
    torch.manual_seed(N)
    x = torch.randn(M, K_).bfloat16()
    w = torch.randn(N, K_).bfloat16()
    ref = x.double() @ w.double().t()
    out = torch.full((M, N), 9.0, device=DEV)
    K.gemv(x.to(DEV), w.to(DEV), out)
    close(out, ref, 3e-6)
    base = torch.randn(M, N)
    acc = base.clone().to(DEV)
    K.gemv(x.to(DEV), w.to(DEV), acc, mode=K.TC_ACCUMULATE)
    close(acc, ref + base.double(), 3e-6)
    I = 19008
    g, u = (torch.randn(I, K_) * 0.2).bfloat16(), (torch.randn(I, K_) * 0.2).bfloat16()
    outs = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    K.gemv(x.to(DEV), interleave(g, u, 64).to(DEV), outs, mode=K.TC_SILU_MUL, pair=64)
    close(outs, P.silu(x.double() @ g.double().t()) * (x.double() @ u.double().t()), 4e-3)


# ------------------------------------------------------------------ prefill attention on tcgen05 (head 64)
def flash_tc_fn(K):
    def fn(q, k_pool, v_pool, out, meta, nh, nkv, hd, window, scale):
        assert K.flash_tc_supported(q, k_pool, nh, nkv, hd, meta.page_size, window)
        n_tiles = sum((c + 127) // 128 for c in meta.new_counts)
        K.flash_prefill_tc(q, k_pool, v_pool, out, meta, meta.seq_start, len(meta.new_counts), n_tiles, nh, nkv, hd,
                           window, scale)
        K.check_status(DEV)
    return fn


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("nh,nkv", [(8, 2), (4, 4), (3, 1), (32, 8)])
def test_flash_prefill_tc(K, nh, nkv, hd):
    fn = flash_tc_fn(K)
    attention_case(K, fn, nh, nkv, hd, torch.bfloat16, [7, 1, 65, 33], [0, 199, 64, 31], None, nh, 6e-3)
    attention_case(K, fn, nh, nkv, hd, torch.bfloat16, [300, 64, 128, 129], [0, 0, 100, 27], None, nh + 2, 6e-3)
    attention_case(K, fn, nh, nkv, hd, torch.bfloat16, [1, 1, 1], [0, 63, 300], None, nh + 1, 6e-3)


@pytest.mark.parametrize("length,needle", [(700, 3), (700, 640), (129, 64), (64, 63), (1000, 0), (65, 64), (257, 128)])
def test_flash_prefill_tc_finds_a_far_key(K, length, needle):
    out, v = needle_case(K, flash_tc_fn(K), torch.bfloat16, length, needle)
    for h in range(4):
        assert torch.allclose(out[h], v[needle, h // 2], atol=2e-2), f"head {h} missed key {needle} of {length}"


@pytest.mark.parametrize("hd", [64, 128])
def test_flash_prefill_tc_ignores_junk_beyond_the_sequence(K, hd):
    attention_case(K, flash_tc_fn(K), 4, 2, hd, torch.bfloat16, [70], [0], None, 5, 6e-3)
    attention_case(K, flash_tc_fn(K), 4, 2, hd, torch.bfloat16, [200, 3], [0, 190], None, 6, 6e-3)


@pytest.mark.parametrize("hd", [64, 128])
def test_flash_prefill_tc_repeats_bit_for_bit(K, hd):
    """Nothing in the kernel depends on timing: many launches on the same inputs (ragged lengths, many heads, so that
    CTAs and row warps finish in every order) give the same bits, and those of the first launch are right."""
    torch.manual_seed(5)
    nh, nkv = 16, 4
    new_counts, before = [300, 77, 129, 513], [0, 50, 0, 100]
    meta = KH.paged_meta(new_counts, before, DEV, 9)
    qs = [torch.randn(t, nh, hd).bfloat16().float() for t in meta.total_len]
    ks = [torch.randn(t, nkv, hd).bfloat16().float() for t in meta.total_len]
    vs = [torch.randn(t, nkv, hd).bfloat16().float() for t in meta.total_len]
    k_pool, v_pool = KH.fill_cache(meta, ks, vs, nkv, hd, torch.bfloat16, DEV)
    q = torch.cat([qb[-n:] for qb, n in zip(qs, new_counts)], 0).reshape(-1, nh * hd).bfloat16().to(DEV)
    fn = flash_tc_fn(K)
    first = torch.empty_like(q)
    fn(q, k_pool, v_pool, first, meta, nh, nkv, hd, None, 1.0 / math.sqrt(hd))
    close(first, KH.plain_attention_rows(qs, ks, vs, new_counts), 6e-3, "first launch")
    for i in range(300):
        out = torch.empty_like(q)
        fn(q, k_pool, v_pool, out, meta, nh, nkv, hd, None, 1.0 / math.sqrt(hd))
        assert torch.equal(out, first), f"launch {i + 2} differs from the first"


@pytest.mark.parametrize("hd", [64, 128])
def test_flash_prefill_tc_reference_maximum_moves_late(K, hd):
    """Scores that keep growing along the keys: the row's reference maximum has to move (and the output so far be
    rescaled) in every block, also late ones; random inputs alone would move it once."""
    torch.manual_seed(11)
    nh = nkv = 2
    L = 640
    q = torch.randn(L, nh, hd) * 0.1
    k = torch.randn(L, nkv, hd) * 0.1
    v = torch.randn(L, nkv, hd)
    s = math.sqrt(hd)
    q[:, :, 0] = s                                    # score of key j = 0.6 j: 38 more per block of 64 keys
    k[:, :, 0] = 0.6 * torch.arange(L).float()[:, None]
    q, k, v = (x.bfloat16().float() for x in (q, k, v))
    meta = KH.paged_meta([L], [0], DEV, 3)
    k_pool, v_pool = KH.fill_cache(meta, [k], [v], nkv, hd, torch.bfloat16, DEV)
    qd = q.reshape(L, nh * hd).bfloat16().to(DEV)
    out = torch.empty_like(qd)
    flash_tc_fn(K)(qd, k_pool, v_pool, out, meta, nh, nkv, hd, None, 1.0 / s)
    ref = KH.plain_attention_rows([q], [k], [v], [L])
    close(out, ref, 2e-2, "growing scores")


def test_gather_i32(K):
    src = torch.arange(100, 140, dtype=torch.int32, device=DEV)
    idx = torch.tensor([3, 0, 39, 7, 7, -1, 40], dtype=torch.int32, device=DEV)
    dst = torch.full((7,), -5, dtype=torch.int32, device=DEV)
    K.gather_i32(src, idx, dst)
    assert dst.tolist() == [103, 100, 139, 107, 107, 0, 0]          # rows outside the source give 0


# ------------------------------------------------------------------ no kernel's result depends on timing
@pytest.mark.parametrize("which", ["flash_prefill", "flash_decode_fused", "flash_decode_two_kernels"])
def test_attention_kernels_repeat_bit_for_bit(K, which):
    torch.manual_seed(8)
    nh, nkv, hd = 8, 2, 64
    if which == "flash_prefill":
        new_counts, before, fn = [300, 77, 129], [0, 50, 0], flash_prefill_fn(K)
    else:
        new_counts, before = [1, 1, 1, 1], [0, 700, 64, 333]
        fn = flash_decode_fn(K, 2, which == "flash_decode_fused")
    meta = KH.paged_meta(new_counts, before, DEV, 4)
    qs = [torch.randn(t, nh, hd).bfloat16().float() for t in meta.total_len]
    ks = [torch.randn(t, nkv, hd).bfloat16().float() for t in meta.total_len]
    vs = [torch.randn(t, nkv, hd).bfloat16().float() for t in meta.total_len]
    k_pool, v_pool = KH.fill_cache(meta, ks, vs, nkv, hd, torch.bfloat16, DEV)
    q = torch.cat([qb[-n:] for qb, n in zip(qs, new_counts)], 0).reshape(-1, nh * hd).bfloat16().to(DEV)
    first = torch.empty_like(q)
    fn(q, k_pool, v_pool, first, meta, nh, nkv, hd, None, 1.0 / math.sqrt(hd))
    for i in range(20):
        out = torch.empty_like(q)
        fn(q, k_pool, v_pool, out, meta, nh, nkv, hd, None, 1.0 / math.sqrt(hd))
        assert torch.equal(out, first), f"{which}: launch {i + 2} differs from the first"


@pytest.mark.parametrize("M,N,K_,bn", [(300, 520, 264, 128), (2048, 512, 2048, 256), (64, 3072, 2048, 128), (17, 2048, 8192, 128),
                                       (1000, 3072, 264, 192)])
def test_tc_gemm_repeats_bit_for_bit(K, M, N, K_, bn):
    torch.manual_seed(3)
    a = torch.randn(M, K_).bfloat16().to(DEV)
    w = torch.randn(N, K_).bfloat16().to(DEV)
    base = torch.randn(M, N, device=DEV)
    first = base.clone()
    K.tc_gemm(a, w, first, mode=K.TC_ACCUMULATE, bn=bn)
    for i in range(10):
        out = base.clone()
        K.tc_gemm(a, w, out, mode=K.TC_ACCUMULATE, bn=bn)
        assert torch.equal(out, first), f"launch {i + 2} differs from the first"
    K.check_status(DEV)


@pytest.mark.parametrize("M,N,K_", [(8, 3072, 2048), (16, 2048, 8192), (3, 100, 200)])
def test_gemv_repeats_bit_for_bit(K, M, N, K_):
    torch.manual_seed(4)
    x = torch.randn(M, K_).bfloat16().to(DEV)
    w = torch.randn(N, K_).bfloat16().to(DEV)
    base = torch.randn(M, N, device=DEV)
    first = base.clone()
    K.gemv(x, w, first, K.TC_ACCUMULATE)
    for i in range(10):
        out = base.clone()
        K.gemv(x, w, out, K.TC_ACCUMULATE)
        assert torch.equal(out, first), f"launch {i + 2} differs from the first"


# ------------------------------------------------------------------ the greedy head: argmax without logits
def _head_argmax(K, x, w):
    M, N = x.shape[0], w.shape[0]
    n_cand = K.head_argmax_candidates(M, N)
    cand = torch.full((M, n_cand, 2), float("nan"), dtype=torch.float32, device=DEV)
    out = torch.full((M,), -7, dtype=torch.int32, device=DEV)
    K.head_argmax(x, w, cand, out)
    return out.cpu()


@pytest.mark.parametrize("M", [1, 3, 8, 16, 17, 33, 64])
@pytest.mark.parametrize("N,Kd", [(333, 72), (1000, 200), (5000, 512), (128256, 256)])
def test_head_argmax_equals_the_argmax_of_the_logits(K, M, N, Kd):
    torch.manual_seed(M * 1000 + N)
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    w = torch.randn(N, Kd, device=DEV).bfloat16()
    logits = x.double() @ w.double().t()
    got = _head_argmax(K, x, w)
    want = logits.argmax(dim=1).cpu()
    top2 = logits.topk(2, dim=1).values
    for m in range(M):
        # the product's float32 sums may order two logits that lie within rounding of each other differently
        if int(got[m]) != int(want[m]):
            assert float(top2[m, 0] - logits[m, int(got[m])]) <= 1e-3 * float(top2[m, 0].abs()), (m, int(got[m]), int(want[m]))


@pytest.mark.parametrize("M", [2, 16, 40])
def test_head_argmax_takes_the_lowest_of_equal_maxima(K, M):
    """Equal maxima in rows that different lanes, warps, tiles and CTAs own: the lowest index wins, as a serial scan
    with a strict ``>`` chooses (crates/spissa-runtime/src/ops.rs:309-324, streaming/argmax.rs:85-97)."""
    N, Kd = 20000, 64
    torch.manual_seed(3)
    w = (torch.randn(N, Kd, device=DEV) * 0.01).bfloat16()
    x = torch.zeros(M, Kd, device=DEV).bfloat16()
    x[:, 0] = 1.0
    twins = [[5, 6], [3, 5 + 8], [7, 40], [130, 129], [9000, 31], [19999, 17000, 12345], [256, 128], [1, 0]]
    for m in range(M):
        rows = twins[m % len(twins)]
        wm = w.clone()
        wm[:, 0] = 0.0
        for r in rows:
            wm[r] = 0.0
            wm[r, 0] = 2.0                      # exactly equal logits, larger than all others
        got = _head_argmax(K, x[m:m + 1].expand(M, Kd).contiguous(), wm)
        assert got.tolist() == [min(rows)] * M, (rows, got.tolist())


def test_head_argmax_ignores_nan_and_rows_beyond_the_table(K):
    N, Kd = 1003, 64                            # the last tile of 8 and of 128 rows is ragged
    torch.manual_seed(5)
    w = torch.randn(N, Kd, device=DEV).bfloat16()
    w[77] = float("nan")
    for M in (4, 20):
        x = torch.randn(M, Kd, device=DEV).bfloat16()
        logits = x.double() @ w.double().t()
        logits[:, 77] = -float("inf")
        assert torch.equal(_head_argmax(K, x, w), logits.argmax(dim=1).cpu().int())


# ------------------------------------------------------------------ products with fused epilogues
# The tile kernel (tc_gemm, prompt steps above 128 tokens; its width argument is the tile width) and the kernel that
# streams the weights (tc_stream, 17 to 128 tokens; width 0, or the block of gate rows) have the same epilogues.
def fused_call(K, bn):
    """(the fused product, sums of squares per row it writes for N columns) for tile width ``bn``; 0: tc_stream."""
    if bn:
        return (lambda a, w, out, mode, pair=0, **kw: K.tc_gemm_fused(a, w, out, mode, 2 * pair if pair else bn, **kw),
                lambda N: K.tc_gemm_n_tiles(N, bn))
    return (lambda a, w, out, mode, pair=0, **kw: K.tc_stream_fused(a, w, out, mode, pair, **kw), K.tc_stream_n_tiles)


@pytest.mark.parametrize("M,N,Kd,bn", [(300, 520, 264, 128), (129, 2048, 512, 256), (513, 1160, 128, 192), (2048, 256, 2048, 256),
                                       (1100, 1160, 264, 128), (1300, 520, 512, 192),
                                       (17, 520, 264, 0), (64, 2048, 8192, 0), (33, 1160, 128, 0), (128, 256, 2048, 0),
                                       (100, 2048, 2048, 0), (1, 200, 72, 0)])
def test_tc_gemm_accumulate_prepares_the_next_norm(K, M, N, Kd, bn):
    """C += A·Wᵀ, and in the same epilogue C ⊙ w_next in bfloat16 and the rows' sums of squares per tile."""
    fused, n_tiles = fused_call(K, bn)
    torch.manual_seed(M + N)
    a = (torch.randn(M, Kd, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, Kd, device=DEV) * 0.1).bfloat16()
    c0 = torch.randn(M, N, device=DEV)
    next_w = (1 + 0.2 * torch.randn(N, device=DEV)).bfloat16()
    c = c0.clone()
    xw = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    ssq = torch.full((M, n_tiles(N)), float("nan"), device=DEV)
    fused(a, w, c, K.TC_ACCUMULATE, xw=xw, next_w=next_w, ssq_out=ssq)
    ref = c0.double() + a.double() @ w.double().t()
    close(c, ref, 2e-5, "residual")
    close(xw.float(), ref * next_w.double(), 6e-3, "residual times the next norm's weight")
    close(ssq.sum(1), (ref ** 2).sum(1), 2e-5, "sums of squares")
    # the consumer: a product on xw whose result is scaled by 1/rms equals the product on the normed rows
    w2 = (torch.randn(384, N, device=DEV) * 0.1).bfloat16()
    out = torch.empty(M, 384, dtype=torch.bfloat16, device=DEV)
    fused_call(K, 128 if bn else 0)[0](xw, w2, out, K.TC_STORE, row_ssq=ssq, norm_width=N, eps=1e-5)
    normed = P.rms_norm(ref, next_w.double().cpu().to(ref.device), 1e-5)
    close(out.float(), normed @ w2.double().t(), 1.2e-2, "product of the normed rows")
    again = c0.clone()
    xw2, ssq2 = torch.empty_like(xw), torch.empty_like(ssq)
    fused(a, w, again, K.TC_ACCUMULATE, xw=xw2, next_w=next_w, ssq_out=ssq2)
    assert torch.equal(again, c) and torch.equal(xw2, xw) and torch.equal(ssq2, ssq)      # a fixed order of sums


@pytest.mark.parametrize("M,I,H,pair,stream", [(200, 384, 264, 64, False), (1030, 1024, 512, 128, False),
                                               (20, 384, 264, 64, True), (64, 8192, 2048, 128, True), (128, 1024, 512, 128, True)])
def test_tc_gemm_silu_epilogue_with_row_scaling(K, M, I, H, pair, stream):
    fused, _ = fused_call(K, 0 if stream else 2 * pair)
    torch.manual_seed(M)
    x = torch.randn(M, H, device=DEV)
    nw = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16()
    xw = (x * nw.float()).bfloat16()
    ssq = (x.double() ** 2).sum(1, keepdim=True).float()
    gate = (torch.randn(I, H, device=DEV) * 0.1).bfloat16()
    up = (torch.randn(I, H, device=DEV) * 0.1).bfloat16()
    wgu = torch.stack([gate.reshape(I // pair, pair, H), up.reshape(I // pair, pair, H)], dim=1).reshape(2 * I, H).contiguous()
    out = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    fused(xw, wgu, out, K.TC_SILU_MUL, pair, row_ssq=ssq, norm_width=H, eps=1e-6)
    rstd = 1.0 / torch.sqrt(ssq.double() / H + 1e-6)
    g = (xw.double() @ gate.double().t()) * rstd
    u = (xw.double() @ up.double().t()) * rstd
    close(out.float(), P.silu(g) * u, 8e-3, "silu(gate)·up of scaled rows")


@pytest.mark.parametrize("hd,nh,nkv,bn,big", [(64, 6, 2, 128, False), (64, 5, 1, 192, False), (64, 32, 8, 256, False),
                                              (128, 4, 2, 256, False), (128, 3, 1, 128, False),
                                              (64, 6, 2, 128, True), (64, 5, 1, 192, True), (64, 32, 8, 256, True),
                                              (128, 4, 2, 256, True), (128, 3, 1, 128, True),
                                              (64, 6, 2, 0, False), (64, 5, 1, 0, False), (64, 32, 8, 0, False),
                                              (128, 4, 2, 0, False), (128, 3, 1, 0, False)])
def test_tc_gemm_qkv_epilogue_rotates_and_writes_the_cache(K, hd, nh, nkv, bn, big):
    """q = rotate(rstd·x·Wqᵀ) stored, k rotated and v plain written into the pages of each token's position, for
    sequences that start at different lengths in one step."""
    fused, _ = fused_call(K, bn)
    torch.manual_seed(hd + nh)
    H = 264 if bn else 2048
    new_counts, before = ([130, 7, 70], [0, 100, 61]) if bn else ([40, 1, 7, 16], [0, 100, 61, 64])
    if big:
        new_counts, before = [700, 7, 330, 70], [0, 100, 61, 5]          # 1,107 rows: tiles of 256 rows by pairs of CTAs
    T = sum(new_counts)
    meta = KH.paged_meta(new_counts, before, DEV, seed=hd)
    x = torch.randn(T, H, device=DEV)
    nw = (1 + 0.1 * torch.randn(H, device=DEV)).bfloat16()
    xw = (x * nw.float()).bfloat16()
    ssq = (x.double() ** 2).sum(1, keepdim=True).float()
    N = (nh + 2 * nkv) * hd
    w = (torch.randn(N, H, device=DEV) * 0.1).bfloat16()
    inv_freq = P.rope_inv_freq(10000.0, hd).to(DEV)
    cs = torch.empty(T, hd // 2, 2, device=DEV)
    tok_page = torch.empty(T, dtype=torch.int32, device=DEV)
    K.rope_table(meta, inv_freq, hd // 2, cs, tok_page)
    ang = meta.positions.float()[:, None] * inv_freq[None, :]
    assert torch.equal(cs[..., 0], torch.cos(ang)) or float((cs[..., 0] - torch.cos(ang)).abs().max()) < 1e-6
    k_pool = torch.full((meta.n_pages, nkv, 64, hd), 7.0, dtype=torch.bfloat16, device=DEV)
    v_pool = torch.full((meta.n_pages, nkv, 64, hd), -7.0, dtype=torch.bfloat16, device=DEV)
    q = torch.full((T, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    fused(xw, w, None, K.TC_QKV_ROPE, row_ssq=ssq, norm_width=H, eps=1e-5,
          rope=dict(cs=cs, tok_page=tok_page, positions=meta.positions, q_out=q, k_pool=k_pool, v_pool=v_pool,
                              nh=nh, nkv=nkv, hd=hd, page_size=64))
    rstd = 1.0 / torch.sqrt(ssq.double() / H + 1e-5)
    qkv = (xw.double() @ w.double().t()) * rstd
    pos = meta.positions.cpu()
    qr = P.apply_rope(qkv[:, :nh * hd].reshape(T, nh, hd).cpu(), pos, inv_freq.double().cpu())
    kr = P.apply_rope(qkv[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd).cpu(), pos, inv_freq.double().cpu())
    vr = qkv[:, (nh + nkv) * hd:].reshape(T, nkv, hd).cpu()
    close(q.float().reshape(T, nh, hd), qr, 8e-3, "rotated queries")
    kc, vc = k_pool.float().cpu(), v_pool.float().cpu()
    t = 0
    touched = torch.zeros(meta.n_pages, 64, dtype=torch.bool)
    for b, (n, b0) in enumerate(zip(new_counts, before)):
        for i in range(n):
            p = b0 + i
            page, off = meta.rows[b][p // 64], p % 64
            touched[page, off] = True
            assert float((kc[page, :, off] - kr[t]).abs().max()) <= 8e-3 * float(kr.abs().max())
            assert float((vc[page, :, off] - vr[t]).abs().max()) <= 8e-3 * float(vr.abs().max())
            t += 1
    kc, vc = kc.permute(0, 2, 1, 3), vc.permute(0, 2, 1, 3)                              # [page, offset, head, dim]
    assert bool((kc[~touched] == 7.0).all()) and bool((vc[~touched] == -7.0).all())      # nothing else was written
