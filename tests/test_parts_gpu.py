"""Each part of a layer alone against its plain formula, built through the part registry."""
import math
from types import SimpleNamespace

import pytest
import torch

import kernel_harness as KH
from plain import llama_plain as P
from spissa_b200.cache.views import KVLayerView
from spissa_b200.config import PartSpec
from spissa_b200.parts import Runtime, build_part
from spissa_b200.parts.rope import rotary_inv_freq

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
TOLS = {torch.float32: 3e-6, torch.bfloat16: 8e-3}


def close(got, ref, tol, what=""):
    err = float((got.double().cpu() - ref.double().cpu()).abs().max())
    scale = float(ref.double().abs().max()) or 1.0
    assert err <= tol * scale, f"{what}: error {err:.3e} against scale {scale:.3e} (allowed {tol:.1e} of it)"


def bound(role, spec, tensors, dtype):
    part = build_part(role, spec)
    rt = Runtime(DEV, dtype, 64)
    store = torch.float32 if dtype == torch.float32 else torch.bfloat16
    part.bind_all({k: v.to(store).to(DEV) for k, v in tensors.items()}, rt)
    return part


def step_of(meta, T):
    return SimpleNamespace(n_tokens=T, token_seq=meta.token_seq, positions=meta.positions, seq_row=meta.seq_slot,
                           seq_slot=meta.seq_slot, seq_len=meta.seq_len, seq_start=meta.seq_start,
                           n_seqs=len(meta.rows), all_single=all(c == 1 for c in meta.new_counts),
                           host=dict(new_counts=list(meta.new_counts)), max_new=T,
                           max_len=max(meta.total_len))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    torch.manual_seed(0)
    w = 1 + 0.2 * torch.randn(200)
    if dtype == torch.bfloat16:
        w = w.bfloat16().float()
    part = bound("norm", PartSpec("rmsnorm", dict(size=200, eps=1e-3), prefix="n."), {"n.weight": w}, dtype)
    h = torch.randn(11, 200)
    out = part.forward(h.to(DEV))
    assert out.dtype == dtype
    close(out, P.rms_norm(h.double(), w.double(), 1e-3), TOLS[dtype])


def test_rotary_table_matches_plain_formula():
    sc = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
              original_max_position_embeddings=128)
    for theta, rd, scaling in [(10000.0, 16, None), (500000.0, 64, sc), (1e6, 128, dict(rope_type="linear", factor=4.0))]:
        mine = rotary_inv_freq(theta, rd, scaling)
        ref = P.rope_inv_freq(theta, rd, scaling)
        assert mine.dtype == torch.float32 and torch.allclose(mine, ref, rtol=1e-6, atol=0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part_adds_into_the_residual(dtype):
    torch.manual_seed(1)
    H, I, T = 72, 136, 9
    w = {"m.gate_proj.weight": torch.randn(I, H) * 0.2, "m.up_proj.weight": torch.randn(I, H) * 0.2,
         "m.down_proj.weight": torch.randn(H, I) * 0.2}
    if dtype == torch.bfloat16:
        w = {k: v.bfloat16().float() for k, v in w.items()}
    part = bound("ffn", PartSpec("swiglu", dict(hidden_size=H, intermediate_size=I), prefix="m."), w, dtype)
    x = torch.randn(T, H).to(dtype)
    res = torch.randn(T, H)
    got = res.clone().to(DEV)
    part.forward(x.to(DEV), None, got)
    ref = res.double() + P.swiglu(x.double(), {k: v.double() for k, v in w.items()}, "m.")
    close(got, ref, TOLS[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, None), (3, 1, 32, None), (3, 3, 48, 40), (8, 2, 64, None)])
def test_attention_part_prefill_then_decode(dtype, nh, nkv, hd, window):
    """The mixer alone: a ragged first step, then one token each, against whole-sequence attention."""
    torch.manual_seed(nh * 7 + hd)
    H = 80
    w = {"a.q_proj.weight": torch.randn(nh * hd, H) * 0.3, "a.k_proj.weight": torch.randn(nkv * hd, H) * 0.3,
         "a.v_proj.weight": torch.randn(nkv * hd, H) * 0.3, "a.o_proj.weight": torch.randn(H, nh * hd) * 0.1}
    if dtype == torch.bfloat16:
        w = {k: v.bfloat16().float() for k, v in w.items()}
    rope = PartSpec("rotary", dict(theta=10000.0, rotary_dim=hd, scaling=None))
    part = bound("mixer", PartSpec("attention", dict(hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                                                     position=rope, window=window), prefix="a."), w, dtype)
    lens = [70, 5, 129]
    xs = [torch.randn(n, H).to(dtype).float() for n in lens]
    n = dict(nh=nh, nkv=nkv, hd=hd)
    inv = P.rope_inv_freq(10000.0, hd)
    refs = [P.attention_block(x.double(), {k: v.double() for k, v in w.items()}, "a.", n, inv, window=window)
            for x in xs]
    # one page table for the whole life of the three sequences
    meta_all = KH.paged_meta(lens, [0, 0, 0], DEV, seed=3)
    k_pool = torch.zeros(meta_all.n_pages, nkv, 64, hd, dtype=dtype, device=DEV)
    v_pool = torch.zeros_like(k_pool)
    first = [l - 2 for l in lens]
    for new_counts, before in ([first, [0, 0, 0]], [[1, 1, 1], first], [[1, 1, 1], [f + 1 for f in first]]):
        meta = KH.paged_meta(new_counts, before, DEV, seed=3)
        meta.page_table, meta.rows = meta_all.page_table, meta_all.rows
        T = sum(new_counts)
        view = KVLayerView(k_pool, v_pool, meta.page_table, 64, meta.token_seq, meta.positions, meta.seq_slot,
                           window, True)
        x = torch.cat([xb[b0:b0 + c] for xb, b0, c in zip(xs, before, new_counts)], 0).to(dtype).to(DEV)
        res = torch.zeros(T, H, dtype=torch.float32, device=DEV)
        part.forward(x, step_of(meta, T), view, res)
        ref = torch.cat([r[b0:b0 + c] for r, b0, c in zip(refs, before, new_counts)], 0)
        close(res, ref, TOLS[dtype] * 2, f"step with {new_counts}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head_parts(dtype):
    torch.manual_seed(2)
    V, H = 333, 72
    E = torch.randn(V, H)
    if dtype == torch.bfloat16:
        E = E.bfloat16().float()
    emb = bound("embedding", PartSpec("embedding", dict(vocab_size=V, hidden_size=H), prefix="e."), {"e.weight": E}, dtype)
    ids = torch.tensor([5, 332, 0], dtype=torch.int32, device=DEV)
    from types import SimpleNamespace
    assert torch.equal(emb.forward(SimpleNamespace(tokens=ids)).cpu(), E[[5, 332, 0]])
    head = bound("head", PartSpec("lm_head", dict(vocab_size=V, hidden_size=H, tied_to="e.weight"), prefix="h."),
                 {"e.weight": E}, dtype)
    assert head.weight_specs() == []
    x = torch.randn(4, H).to(dtype)
    out = head.forward(x.to(DEV))
    assert out.dtype == torch.float32
    close(out, x.double() @ E.double().t(), 3e-6)
