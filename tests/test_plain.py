"""The plain implementation against fixed points.

The vectors are those of the reference's own unit tests (read as text; the reference is a
Rust project that cannot be compiled here): crates/spissa-runtime/src/ops.rs:473-615 and
crates/spissa-runtime/src/rotary.rs:616-670, :827-851.
"""
import math

import pytest
import torch

from plain import llama_plain as P


def test_embedding_rows():                                     # ops.rs:474-478
    table = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])
    assert P.embedding(table, [2, 0]).flatten().tolist() == [5.0, 6.0, 1.0, 2.0]
    with pytest.raises(ValueError):
        P.embedding(table, [3])


def test_linear_uses_out_in_layout():                          # ops.rs:489-495 (without its bias)
    x = torch.tensor([[1.0, 2.0, 3.0]])
    w = torch.tensor([[1.0, 0.0, 1.0], [0.5, 0.5, 0.5]])
    assert P.linear(x, w).flatten().tolist() == [4.0, 3.0]


def test_rms_norm():                                           # ops.rs:507-513
    out = P.rms_norm(torch.tensor([[3.0, 4.0]]), torch.ones(2), 0.0)
    d = math.sqrt(12.5)
    assert torch.allclose(out, torch.tensor([[3.0 / d, 4.0 / d]]), atol=1e-6)


def test_silu_known_points():                                  # ops.rs:529-534
    assert abs(float(P.silu(torch.tensor(0.0)))) < 1e-6
    assert abs(float(P.silu(torch.tensor(1.0))) - 0.731058) < 1e-5


def test_attention_causal_mask():                              # ops.rs:537-554
    q = torch.tensor([[[1.0, 0.0]], [[0.0, 1.0]]])
    v = torch.tensor([[[10.0, 0.0]], [[0.0, 20.0]]])
    out = P.causal_attention(q, q.clone(), v)
    assert torch.allclose(out[0], torch.tensor([10.0, 0.0]), atol=1e-6)
    assert 3.0 < float(out[1, 0]) < 3.4 and 13.0 < float(out[1, 1]) < 13.7


def test_attention_softmax_is_stable():                        # ops.rs:516-521 through the attention path
    q = torch.tensor([[[1000.0]], [[1001.0]]])
    k = torch.tensor([[[1.0]], [[1.0]]])
    v = torch.tensor([[[0.0]], [[1.0]]])
    out = P.causal_attention(q, k, v)
    assert torch.isfinite(out).all() and abs(float(out[1, 0]) - 0.5) < 1e-6


def test_window_limits_keys():
    T = 6
    q = torch.zeros(T, 1, 2)
    v = torch.arange(T, dtype=torch.float32).reshape(T, 1, 1).repeat(1, 1, 2)
    out = P.causal_attention(q, torch.zeros(T, 1, 2), v, window=2)
    assert torch.allclose(out[:, 0], torch.tensor([0.0, 0.5, 1.5, 2.5, 3.5, 4.5]))


def test_argmax_first_maximum():                               # ops.rs:571-573 and :309-324
    assert P.sample_argmax([0.1, 2.0, 1.9]) == 1
    assert P.sample_argmax([1.0, 3.0, 3.0]) == 1


def test_top_k_one_is_argmax_for_any_seed():                   # ops.rs:609-615
    for seed in (0, 1, 42, 9999):
        assert P.sample_top_k_top_p([0.1, 0.2, 2.0, 1.0], 1.0, 1, 1.0, seed) == 2


def test_same_seed_same_sample():                              # ops.rs:600-606
    a = P.sample_top_k_top_p([0.1, 0.2, 2.0, 1.0], 0.8, 0, 0.95, 1234)
    assert a == P.sample_top_k_top_p([0.1, 0.2, 2.0, 1.0], 0.8, 0, 0.95, 1234) and 0 <= a < 4


def test_seeded_unit_range_and_zero_seed():                    # ops.rs:446-457
    for s in (0, 1, 2, 1234, 2 ** 63):
        assert 0.0 <= P.seeded_unit_f32(s) < 1.0
    assert P.seeded_unit_f32(0) == P.seeded_unit_f32(0x9E3779B97F4A7C15)


def test_rope_rotate_half_against_manual_loop():               # rotary.rs:616-670
    hd, rd, theta, offset = 8, 4, 10000.0, 3
    x = torch.arange(2 * 2 * hd, dtype=torch.float32).reshape(2, 2, hd) / 7.0
    inv = P.rope_inv_freq(theta, rd)
    out = P.apply_rope(x, torch.arange(2) + offset, inv)
    for t in range(2):
        for h in range(2):
            for i in range(rd // 2):
                ang = (offset + t) * (1.0 / theta ** (2 * i / rd))
                a, b = float(x[t, h, i]), float(x[t, h, i + rd // 2])
                assert abs(float(out[t, h, i]) - (a * math.cos(ang) - b * math.sin(ang))) < 1e-5
                assert abs(float(out[t, h, i + rd // 2]) - (b * math.cos(ang) + a * math.sin(ang))) < 1e-5
            assert torch.equal(out[t, h, rd:], x[t, h, rd:])     # tail dims untouched


def test_llama3_scaling_hits_all_three_branches():
    sc = dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
              original_max_position_embeddings=64)
    base = P.rope_inv_freq(500000.0, 32)
    scaled = P.rope_inv_freq(500000.0, 32, sc)
    lam = 2 * math.pi / base
    kept = lam < 64 / 4.0
    divided = lam > 64 / 1.0
    between = ~kept & ~divided
    assert kept.any() and divided.any() and between.any()
    assert torch.equal(scaled[kept], base[kept])
    assert torch.allclose(scaled[divided], base[divided] / 32.0, rtol=1e-6)
    assert ((scaled[between] < base[between]) & (scaled[between] > base[between] / 32.0)).all()


def test_cached_attention_equals_last_row_of_full():           # rotary.rs:827-851, restated without a cache
    torch.manual_seed(0)
    T, nh, nkv, hd = 7, 4, 2, 8
    q, k, v = torch.randn(T, nh, hd), torch.randn(T, nkv, hd), torch.randn(T, nkv, hd)
    full = P.causal_attention(q, k, v)
    # the last query alone over all keys: build it as a 1-row problem by brute force
    rep = nh // nkv
    for h in range(nh):
        s = (k[:, h // rep] @ q[-1, h]) / math.sqrt(hd)
        p = torch.softmax(s, 0)
        assert torch.allclose(full[-1, h * hd:(h + 1) * hd], p @ v[:, h // rep], atol=1e-6)


def test_model_logits_shape_and_tied_head(tmp_path):
    import tiny
    tiny.make_folder(tiny.TINY_A, tiny.TINY_A_INIT, tmp_path)
    cfg, w = P.read_model_folder(tmp_path)
    assert "lm_head.weight" not in w
    out = P.model_logits(cfg, w, [1, 2, 3])
    assert out.shape == (3, 256)
    # causality: a longer sequence leaves earlier rows alone
    out2 = P.model_logits(cfg, w, [1, 2, 3, 9, 8])
    assert torch.allclose(out, out2[:3], atol=1e-12)
