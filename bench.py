"""Measures decoding and prefill of the Llama-3.2-1B shape with random bfloat16 weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--config 1b|3b|8b] [--batch B]
                    [--context T] [--profile-phases]

Prints ONE JSON line. ``value`` is decoded tokens per second at batch 8 from prompts of
about 2,048 tokens in a cache of 4,096 tokens per sequence, timed on the device with CUDA
events over exactly K decode steps after W warm-up steps; ``e2e`` is the same through the
Python entry point (``Engine.generate``: host token lists in, host token lists out).
``prefill`` is one 2,048-token prompt; ``points`` holds decoding at batch 1 and 64;
``roofline`` compares the decode step with the bytes it has to read. ``--context T`` decodes from prompts of
about T tokens instead (the cache then holds 2T per sequence); the prefill measurement stays at 2,048 tokens.
``--config 3b`` and ``--config 8b`` run the secondary workloads (3B shape: batch 8, prompts uniform in [256, 2048],
256 decode steps, 4,096-token cache per sequence; 8B shape: batch 16, prompts uniform in [512, 4096], 512 steps,
8,192 tokens per sequence) and print the same line. ``--profile-phases`` adds per-phase timings (CUDA events around
the kernel groups of one prompt step and of part-by-part decode steps).
Token ids are synthetic (seeded, uniform over the vocabulary), weights are N(0, 0.02).
Every decode step reads all weights (2.47 GB), far more than the 126 MB L2, so no
flush is needed between timed iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# the Llama 3.2 1B shape: the configuration the headline numbers are quoted on
CONFIG_1B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=16, hidden_size=2048,
    num_attention_heads=32, num_key_value_heads=8, head_dim=64, intermediate_size=8192, vocab_size=128256,
    rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    tie_word_embeddings=True, rms_norm_eps=1e-5, max_position_embeddings=131072)
CONFIG_3B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=28, hidden_size=3072,
    num_attention_heads=24, num_key_value_heads=8, head_dim=128, intermediate_size=8192, vocab_size=128256,
    rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    tie_word_embeddings=True, rms_norm_eps=1e-5, max_position_embeddings=131072)
CONFIG_8B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=32, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=128256,
    rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    tie_word_embeddings=False, rms_norm_eps=1e-5, max_position_embeddings=131072)
# name -> configuration, batch, cache per sequence, prompt lengths (mean of a narrow band, or a uniform range), decode
# steps, extra batch sizes: the headline workload and the two secondary ones
WORKLOADS = {
    "1b": dict(cfg=CONFIG_1B, model="llama-3.2-1b-shape", batch=8, context=4096, prompt=2048, span=None, steps=64, points="1,64"),
    "3b": dict(cfg=CONFIG_3B, model="llama-3.2-3b-shape", batch=8, context=4096, prompt=None, span=(256, 2048), steps=256, points=""),
    "8b": dict(cfg=CONFIG_8B, model="llama-3.1-8b-shape", batch=16, context=8192, prompt=None, span=(512, 4096), steps=512, points=""),
}
CONTEXT = 4096
PROMPT = 2048
SPAN = None                                 # (lowest, highest) prompt length when the workload draws them uniformly
PREFILL_TOKENS = 2048                       # the prefill measurement is always of this many tokens
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            d = json.load(fh)
        out = dict(FALLBACK_PEAKS)
        for k in out:
            if isinstance(d.get(k), (int, float)) and d[k] > 0:
                out[k] = float(d[k])
        out["source"] = "measured"
        return out
    except Exception:
        return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return dict(sm_mhz=sm[len(sm) // 2] if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def model_numbers(cfg, elem_bytes=2):
    H, I, L = cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers
    nh, nkv, hd, V = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.vocab_size
    per_layer = H * nh * hd * 2 + H * nkv * hd * 2 + 3 * H * I
    head = V * H
    return dict(per_layer=per_layer, head=head, kv_bytes_per_token=2 * nkv * hd * elem_bytes * L,
                weight_bytes=(per_layer * L + head) * elem_bytes)


def prefill_flops(cfg, T):
    n = model_numbers(cfg)
    gemm = 2.0 * T * n["per_layer"] * cfg.num_hidden_layers
    attn = 4.0 * (T * (T + 1) / 2) * cfg.head_dim * cfg.num_attention_heads * cfg.num_hidden_layers
    return gemm + attn + 2.0 * n["head"]


def ragged_lengths(batch, seed):
    rng = random.Random(seed)
    if SPAN is not None:
        return [rng.randint(SPAN[0], SPAN[1]) for _ in range(batch)]
    if batch == 1:
        return [PROMPT]
    half = PROMPT // 8
    lens = [PROMPT + rng.randrange(-half, half + 1) for _ in range(batch)]
    lens[0] += PROMPT * batch - sum(lens)         # the mean is PROMPT exactly
    return lens


KERNEL_CASE_LAYERS = 0
KERNEL_CASE_BATCH = 0          # sequences of --kernel-case decode_layers (0: eight)


def kernel_case(name: str, reps: int) -> int:
    """One kernel of the step alone, at the 1B shape, on rotating buffers larger than L2.

    Prints one JSON line with its time and its fraction of the measured peak. This is what the
    ncu summaries under profiles/ were captured from (``--kernel-case NAME --reps 3``).
    """
    import math
    import torch
    from types import SimpleNamespace
    from spissa_b200.csrc import lib as K
    peaks = load_peaks()
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    H, I, V, nh, nkv, hd, T = 2048, 8192, 128256, 32, 8, 64, PROMPT
    bf = torch.bfloat16

    def rnd(*shape):
        return (torch.randn(*shape, device=dev) * 0.05).to(bf)

    flops = bytes_ = 0.0
    if name == "step_b8":
        # eight 2,048-token prompts one after another, then three decode steps at batch 8, kernel by kernel and
        # part by part (no CUDA graph, no one-kernel decode): the launch list of this run is what
        # profiles/step_b8_launches.md summarises
        from spissa_b200 import Engine, LlamaConfig
        eng = Engine.from_config(LlamaConfig.from_dict(CONFIG_1B), seed=0, dtype="bfloat16", max_tokens=8 * CONTEXT,
                                 max_seqs=8, use_graphs=False, fuse_decode=False)
        rng = random.Random(0)
        slots = [eng.acquire() for _ in range(8)]
        for sl in slots:
            eng.step([(sl, [rng.randrange(V) for _ in range(T)], [T - 1])])
        for i in range(3):
            eng.step([(sl, [5 + i], [0]) for sl in slots])
        torch.cuda.synchronize()
        print(json.dumps({"kernel_case": name, "launches": K.launches}))
        return 0
    if name == "prefill":
        # prompts of 2,048 tokens one after another through the engine's own step (the launch list of this run is
        # what profiles/prefill_step_fused_launches.md summarises)
        from spissa_b200 import Engine, LlamaConfig
        cfg = dict(CONFIG_1B)
        if KERNEL_CASE_LAYERS:
            cfg["num_hidden_layers"] = KERNEL_CASE_LAYERS
        eng = Engine.from_config(LlamaConfig.from_dict(cfg), seed=0, dtype="bfloat16", max_tokens=2 * CONTEXT, max_seqs=2)
        rng = random.Random(0)
        times = []
        for i in range(max(2, reps)):
            sl = eng.acquire()
            toks = [rng.randrange(V) for _ in range(T)]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            l0 = K.launches
            e0.record()
            eng.step([(sl, toks, [T - 1])], greedy=True, check=False)
            e1.record()
            torch.cuda.synchronize()
            eng.check()
            times.append(e0.elapsed_time(e1))
            eng.release(sl)
        print(json.dumps({"kernel_case": name, "layers": cfg["num_hidden_layers"], "ms": [round(t, 3) for t in times],
                          "launches_per_step": K.launches - l0}))
        return 0
    if name == "decode_layers":
        # the one-kernel decode path alone: eight 2,048-token prompts, then decode steps launched one by one; the
        # last one records the global timer as CTA 0 enters and leaves each grid barrier (phase times per layer)
        import ctypes
        from spissa_b200 import Engine, LlamaConfig
        cfg = dict(CONFIG_1B)
        if KERNEL_CASE_LAYERS:
            cfg["num_hidden_layers"] = KERNEL_CASE_LAYERS
        nl = cfg["num_hidden_layers"]
        n_seqs = KERNEL_CASE_BATCH or 8
        eng = Engine.from_config(LlamaConfig.from_dict(cfg), seed=0, dtype="bfloat16", max_tokens=n_seqs * CONTEXT,
                                 max_seqs=n_seqs, use_graphs=False)
        rng = random.Random(0)
        slots = [eng.acquire() for _ in range(n_seqs)]
        for sl in slots:
            eng.step([(sl, [rng.randrange(V) for _ in range(T)], [T - 1])])
        for i in range(max(1, reps - 1)):
            eng.step([(sl, [5 + i], [0]) for sl in slots])
        trace = torch.zeros(1024, dtype=torch.int64, device=dev)
        lib = K.load("decode_layers")
        lib.sp_decode_layers_set_trace(ctypes.c_void_p(trace.data_ptr()))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.step([(sl, [9], [0]) for sl in slots], greedy=True)
        e1.record()
        torch.cuda.synchronize()
        lib.sp_decode_layers_set_trace(ctypes.c_void_p(0))
        K.check_status(dev)
        t = trace.cpu().tolist()
        # six grid barriers per layer, or five where the chunks are combined inside the attention phase by CTA pairs
        # (the last layer's last barrier does not exist: the kernel ends there)
        per_layer = ["qkv", "attention", "combine", "output projection", "gate/up", "down"]
        if t[2 * 6 * nl] == 0:
            per_layer = ["qkv", "attention+combine", "output projection", "gate/up", "down"]
        names = ["input statistics"] + per_layer * nl
        work, wait = {}, {}
        for e in range(1, len(per_layer) * nl + 1):              # barrier e: entered at t[2e], left at t[2e + 1]
            work.setdefault(names[e - 1], []).append(t[2 * e] - t[2 * e - 1])
            wait.setdefault(names[e - 1], []).append(t[2 * e + 1] - t[2 * e])
        med = lambda v: sorted(v)[len(v) // 2] / 1e3
        last = len(per_layer) * nl                                # behind the last layer: the final norm and the head, if the kernel ran them
        head_us = round((t[1023] - t[2 * last + 1]) / 1e3, 2) if t[2 * last + 1] else None
        print(json.dumps({"kernel_case": name, "layers": nl, "sequences": n_seqs, "kernel_us": round((t[1023] - t[1]) / 1e3, 1),
                          "head_us": head_us,
                          "step_ms_with_host": round(e0.elapsed_time(e1), 3),
                          "phase_us_median": {k: round(med(v), 2) for k, v in work.items()},
                          "barrier_us_median": {k: round(med(v), 2) for k, v in wait.items()},
                          "fused_steps": eng.model._fused.runs if eng.model._fused else 0}))
        return 0
    if name in ("gemm_qkv", "gemm_o", "gemm_gate_up", "gemm_down"):
        from spissa_b200.parts.linear import tile_width
        N, Kd, mode, bn = {"gemm_qkv": (3072, H, K.TC_STORE, tile_width(T, 3072, 148)), "gemm_o": (H, H, K.TC_ACCUMULATE, tile_width(T, H, 148)),
                           "gemm_gate_up": (2 * I, H, K.TC_SILU_MUL, 256),
                           "gemm_down": (H, I, K.TC_ACCUMULATE, 256)}[name]
        n_buf = max(2, int(300e6 // (N * Kd * 2)) + 1)
        ws = [rnd(N, Kd) for _ in range(n_buf)]
        a = rnd(T, Kd)
        out = torch.zeros(T, N // 2 if mode == K.TC_SILU_MUL else N,
                          dtype=torch.float32 if mode == K.TC_ACCUMULATE else bf, device=dev)
        run = lambda i: K.tc_gemm(a, ws[i % n_buf], out, mode, bn)
        flops = 2.0 * T * N * Kd
    elif name in ("fused_qkv", "fused_o", "fused_gate_up", "fused_down"):
        # the same products with the epilogues of a fused prompt step (engine/fused_prefill.py)
        from spissa_b200.parts.linear import tile_width
        N, Kd = {"fused_qkv": (3072, H), "fused_o": (H, H), "fused_gate_up": (2 * I, H), "fused_down": (H, I)}[name]
        n_buf = max(2, int(300e6 // (N * Kd * 2)) + 1)
        ws = [rnd(N, Kd) for _ in range(n_buf)]
        a = rnd(T, Kd)
        ssq = torch.rand(T, 8, device=dev) + 1.0
        flops = 2.0 * T * N * Kd
        if name == "fused_qkv":
            bn = tile_width(T, N, 148)
            pages = T // 64
            kp, vp = rnd(pages, nkv, 64, hd), rnd(pages, nkv, 64, hd)
            q = torch.empty(T, nh * hd, dtype=bf, device=dev)
            cs = torch.rand(T, hd // 2, 2, device=dev)
            pos = torch.arange(T, dtype=torch.int32, device=dev)
            tok_page = (pos // 64).int()
            rope = dict(cs=cs, tok_page=tok_page, positions=pos, q_out=q, k_pool=kp, v_pool=vp, nh=nh, nkv=nkv, hd=hd, page_size=64)
            run = lambda i: K.tc_gemm_fused(a, ws[i % n_buf], None, K.TC_QKV_ROPE, bn, row_ssq=ssq, norm_width=H, eps=1e-5, rope=rope)
        elif name == "fused_gate_up":
            out = torch.empty(T, I, dtype=bf, device=dev)
            run = lambda i: K.tc_gemm_fused(a, ws[i % n_buf], out, K.TC_SILU_MUL, 256, row_ssq=ssq, norm_width=H, eps=1e-5)
        else:
            bn = tile_width(T, N, 148)
            out = torch.zeros(T, N, device=dev)
            xw = torch.empty(T, N, dtype=bf, device=dev)
            nw = rnd(N)
            so = torch.empty(T, K.tc_gemm_n_tiles(N, bn), device=dev)
            run = lambda i: K.tc_gemm_fused(a, ws[i % n_buf], out, K.TC_ACCUMULATE, bn, xw=xw, next_w=nw, ssq_out=so)
    elif name in ("stream_qkv", "stream_o", "stream_gate_up", "stream_down"):
        # the products of a decode step of 64 sequences: tc_stream.cu
        N, Kd, mode, pair = {"stream_qkv": (3072, H, K.TC_STORE, 0), "stream_o": (H, H, K.TC_ACCUMULATE, 0),
                             "stream_gate_up": (2 * I, H, K.TC_SILU_MUL, 128),
                             "stream_down": (H, I, K.TC_ACCUMULATE, 0)}[name]
        n_buf = max(2, int(300e6 // (N * Kd * 2)) + 1)
        ws = [rnd(N, Kd) for _ in range(n_buf)]
        x = rnd(64, Kd)
        out = torch.zeros(64, N // 2 if mode == K.TC_SILU_MUL else N,
                          dtype=torch.float32 if mode == K.TC_ACCUMULATE else bf, device=dev)
        run = lambda i: K.tc_stream(x, ws[i % n_buf], out, mode, pair)
        bytes_ = N * Kd * 2.0
    elif name in ("stream_fused_qkv", "stream_fused_o", "stream_fused_gate_up", "stream_fused_down"):
        # the same products of 64 tokens with the fused epilogues (engine/fused_prefill.py, 17 to 64 tokens)
        N, Kd = {"stream_fused_qkv": (3072, H), "stream_fused_o": (H, H), "stream_fused_gate_up": (2 * I, H),
                 "stream_fused_down": (H, I)}[name]
        M = 64
        n_buf = max(2, int(300e6 // (N * Kd * 2)) + 1)
        ws = [rnd(N, Kd) for _ in range(n_buf)]
        a = rnd(M, Kd)
        ssq = torch.rand(M, 16, device=dev) + 1.0
        bytes_ = N * Kd * 2.0
        if name == "stream_fused_qkv":
            kp, vp = rnd(M, nkv, 64, hd), rnd(M, nkv, 64, hd)          # every token in a page of its own: a decode step
            q = torch.empty(M, nh * hd, dtype=bf, device=dev)
            cs = torch.rand(M, hd // 2, 2, device=dev)
            pos = torch.full((M,), 2047, dtype=torch.int32, device=dev)
            tok_page = torch.arange(M, dtype=torch.int32, device=dev)
            rope = dict(cs=cs, tok_page=tok_page, positions=pos, q_out=q, k_pool=kp, v_pool=vp, nh=nh, nkv=nkv, hd=hd, page_size=64)
            run = lambda i: K.tc_stream_fused(a, ws[i % n_buf], None, K.TC_QKV_ROPE, 0, row_ssq=ssq, norm_width=H, eps=1e-5, rope=rope)
        elif name == "stream_fused_gate_up":
            out = torch.empty(M, I, dtype=bf, device=dev)
            run = lambda i: K.tc_stream_fused(a, ws[i % n_buf], out, K.TC_SILU_MUL, 128, row_ssq=ssq, norm_width=H, eps=1e-5)
        else:
            out = torch.zeros(M, N, device=dev)
            xw = torch.empty(M, N, dtype=bf, device=dev)
            nw = rnd(N)
            so = torch.empty(M, K.tc_stream_n_tiles(N), device=dev)
            run = lambda i: K.tc_stream_fused(a, ws[i % n_buf], out, K.TC_ACCUMULATE, 0, xw=xw, next_w=nw, ssq_out=so)
    elif name in ("gemv_qkv", "gemv_o", "gemv_gate_up", "gemv_down", "gemv_head"):
        N, Kd, mode = {"gemv_qkv": (3072, H, K.TC_STORE), "gemv_o": (H, H, K.TC_ACCUMULATE),
                       "gemv_gate_up": (2 * I, H, K.TC_SILU_MUL), "gemv_down": (H, I, K.TC_ACCUMULATE),
                       "gemv_head": (V, H, K.TC_STORE)}[name]
        n_buf = max(2, int(300e6 // (N * Kd * 2)) + 1)
        ws = [rnd(N, Kd) for _ in range(n_buf)]
        x = rnd(8, Kd)
        out = torch.zeros(8, N // 2 if mode == K.TC_SILU_MUL else N,
                          dtype=bf if mode == K.TC_SILU_MUL else torch.float32, device=dev)
        run = lambda i: K.gemv(x, ws[i % n_buf], out, mode, 128)
        bytes_ = N * Kd * 2.0
    elif name in ("flash_prefill", "flash_prefill_tc", "flash_decode", "flash_decode_b64", "flash_prefill_128",
                  "flash_prefill_tc_128"):
        if name.endswith("_128"):          # the 8B shape's attention: 32 heads of 128, 8 kv heads
            hd, name = 128, name[:-4]
        decode_batch = {"flash_decode": 8, "flash_decode_b64": 64}.get(name, 0)
        B = decode_batch or 1
        n_new = 1 if decode_batch else T
        pages = B * (T // 64)
        n_buf = 320 // decode_batch if decode_batch else 1    # 40 x 8.4 MB (5 x 67 MB) of keys and values > L2
        pools = [(rnd(pages, nkv, 64, hd), rnd(pages, nkv, 64, hd)) for _ in range(n_buf)]
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(B, T // 64)
        ar = torch.arange(B, dtype=torch.int32, device=dev)
        meta = SimpleNamespace(page_table=table, page_size=64, seq_slot=ar,
                               positions=(torch.arange(n_new, dtype=torch.int32, device=dev) + (T - n_new)).repeat(B),
                               token_seq=ar.repeat_interleave(n_new))
        q = rnd(B * n_new, nh * hd)
        out = torch.empty_like(q)
        scale = 1.0 / math.sqrt(hd)
        if name == "flash_prefill":
            seq_start = torch.tensor([0, T], dtype=torch.int32, device=dev)
            run = lambda i: K.flash_prefill(q, pools[0][0], pools[0][1], out, meta, seq_start, 1, T // 64, nh, nkv,
                                            hd, None, scale)
            flops = 4.0 * (T * (T + 1) / 2) * hd * nh
        elif name == "flash_prefill_tc":
            seq_start = torch.tensor([0, T], dtype=torch.int32, device=dev)
            run = lambda i: K.flash_prefill_tc(q, pools[0][0], pools[0][1], out, meta, seq_start, 1, T // 128, nh, nkv,
                                               hd, None, scale)
            flops = 4.0 * (T * (T + 1) / 2) * hd * nh
        else:
            seq_len = torch.full((B,), T, dtype=torch.int32, device=dev)
            ct, nc = K.flash_decode_plan(B, nkv, T)
            scratch = torch.empty(K.flash_decode_scratch_floats(B, nh, hd, nc), device=dev)
            run = lambda i: K.flash_decode(q, pools[i % n_buf][0], pools[i % n_buf][1], out, meta, seq_len, nh, nkv,
                                           hd, None, scale, ct, nc, scratch)
            bytes_ = B * T * nkv * hd * 2 * 2.0
    elif name in ("sample_b8", "sample_b64", "argmax_b8"):
        # the sampler on rows of 128,256 logits (standard deviation 4 after the temperature): temperature 0.8, top-p 0.95
        B = 64 if name.endswith("b64") else 8
        logits = [torch.randn(B, V, device=dev) * 3.2 for _ in range(4)]
        u = torch.rand(B, device=dev)
        out = torch.empty(B, dtype=torch.int32, device=dev)
        scratch = torch.empty(K.sample_scratch_keys(B, V), dtype=torch.int64, device=dev)
        if name.startswith("argmax"):
            run = lambda i: K.argmax_rows(logits[i % 4], out)
        else:
            run = lambda i: K.sample_rows(logits[i % 4], 0.8, 0, 0.95, u, scratch, out)
        bytes_ = B * V * 4.0
    else:
        print("unknown kernel case", name)
        return 2
    for i in range(3):
        run(i)
    torch.cuda.synchronize()
    # the launches are replayed from a CUDA graph so that the host's launch cost is not in the number
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(reps):
            run(3 + i)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    K.check_status(dev)
    us = e0.elapsed_time(e1) * 1000.0 / reps
    line = {"kernel_case": name, "us": round(us, 2), "reps": reps, "peaks": peaks["source"]}
    if flops:
        line.update(tflops=round(flops / us / 1e6, 1), frac=round(flops / us / 1e6 / peaks["bf16_tflops"], 4))
    if bytes_:
        line.update(gbs=round(bytes_ / us / 1e3, 1), frac=round(bytes_ / us / 1e3 / peaks["hbm_gbs"], 4))
    print(json.dumps(line))
    return 0


def main() -> int:
    global PROMPT, CONTEXT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed decode steps (default: the workload's: 64, 256 or 512)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="1b", choices=sorted(WORKLOADS), help="the headline workload (1b) or a secondary one")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="float32: the true 32-bit path of the whole model (FFMA products, no tensor cores); its prefill "
                         "fraction is of the nominal FFMA rate (148 SMs x 128 lanes x 2 x the maximum SM clock)")
    ap.add_argument("--context", type=int, default=None,
                    help="mean prompt length of the decode runs (the cache holds twice as much per sequence)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--points", default=None, help="extra decode batch sizes, comma separated ('' = none)")
    ap.add_argument("--profile-phases", action="store_true", dest="profile_phases",
                    help="add per-phase timings of one prompt step and of part-by-part decode steps")
    ap.add_argument("--kernel-case", default=None,
                    help="time one kernel alone (gemm_qkv|gemm_o|gemm_gate_up|gemm_down|gemv_qkv|gemv_o|gemv_gate_up|"
                         "gemv_down|gemv_head|stream_qkv|stream_o|stream_gate_up|stream_down|stream_fused_qkv|stream_fused_o|stream_fused_gate_up|stream_fused_down|flash_prefill[_128]|flash_prefill_tc[_128]|flash_decode[_b64]|sample_b8|sample_b64|argmax_b8|decode_layers|step_b8|prefill|fused_qkv|fused_o|fused_gate_up|fused_down) instead of the step")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--case-layers", type=int, default=0, help="layers of the model in --kernel-case decode_layers (0: all)")
    args = ap.parse_args()
    if args.kernel_case:
        global KERNEL_CASE_LAYERS, KERNEL_CASE_BATCH
        KERNEL_CASE_LAYERS = args.case_layers
        KERNEL_CASE_BATCH = args.batch or 0
        return kernel_case(args.kernel_case, args.reps)

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "Erik-cpu-create/spissa is a Rust CPU project with no Python package "
                          "(pip: neither setup.py nor pyproject.toml) and no Rust toolchain is installed"}))
        return 0
    if args.gpus != 1:
        print("bench.py: this library runs on ONE GPU; --gpus %d is not supported" % args.gpus)
        return 2
    if args.warmup < 3:
        args.warmup = 3
    global SPAN
    work = WORKLOADS[args.config]
    args.steps = args.steps or work["steps"]
    args.batch = args.batch or work["batch"]
    args.points = work["points"] if args.points is None else args.points
    CONTEXT, SPAN = work["context"], work["span"]
    PROMPT = work["prompt"] or (SPAN[0] + SPAN[1]) // 2
    if args.context is not None and args.context != PROMPT:
        SPAN = None
        if args.context < 64:
            print("bench.py: --context must be at least 64")
            return 2
        PROMPT, CONTEXT = args.context, max(2 * args.context, PREFILL_TOKENS + 64)

    import torch
    from spissa_b200 import Engine, LlamaConfig, SamplingParams
    from spissa_b200.csrc import lib

    peaks = load_peaks()
    cfg_dict = dict(work["cfg"])
    full_layers = cfg_dict["num_hidden_layers"]
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    cfg = LlamaConfig.from_dict(cfg_dict)
    fp32 = args.dtype == "float32"
    nums = model_numbers(cfg, 4 if fp32 else 2)
    points = [int(x) for x in args.points.split(",") if x.strip()]
    max_batch = max([args.batch] + points)
    torch.cuda.set_device(0)
    engine = Engine.from_config(cfg, seed=0, dtype=args.dtype, max_tokens=max_batch * CONTEXT,
                                max_seqs=max_batch, device="cuda:0")
    rng = random.Random(1234)
    V = cfg.vocab_size

    def prompts_for(batch):
        return [[rng.randrange(V) for _ in range(n)] for n in ragged_lengths(batch, 99 + batch)]

    from spissa_b200.sampling import Sampler
    sampler = Sampler(engine.device)
    greedy = SamplingParams()

    def decode_run(batch, steps, warmup):
        """Device-timed decode steps at ``batch`` after a ragged prefill; returns (ms per step, kv tokens, launches)."""
        prompts = prompts_for(batch)
        slots = [engine.acquire() for _ in range(batch)]
        # prompts go in as chunks so that a step never carries more than 8k tokens
        fed = [0] * batch
        while any(f < len(p) for f, p in zip(fed, prompts)):
            ents, room = [], 8192
            for b in range(batch):
                n = min(len(prompts[b]) - fed[b], room)
                if n > 0:
                    ents.append((slots[b], prompts[b][fed[b]:fed[b] + n], []))
                    fed[b] += n
                    room -= n
                if room == 0:
                    break
            engine.step(ents, check=False)
        engine.check()
        toks = [rng.randrange(V) for _ in range(batch)]

        def one():
            # launched back to back: the steps are confirmed (status word read) by ``engine.check()`` after the timing;
            # greedy: the head returns the tokens (no logits are written), as in ``Engine.generate``
            return engine.step([(s, [t], [0]) for s, t in zip(slots, toks)], check=False, greedy=True)

        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        kv_tokens = sum(engine.length(s) for s in slots) + batch * steps // 2
        l0 = lib.launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            one()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        launches = lib.launches - l0
        engine.check()
        for s in slots:
            engine.release(s)
        return ms, kv_tokens, launches, [len(p) for p in prompts]

    # ---------------------------------------------------------------- decode, device timed
    clocks = ClockSampler()
    clocks.start()
    ms_step, kv_tokens, launches, prompt_lens = decode_run(args.batch, args.steps, args.warmup)
    clock_info = clocks.stop()
    value = args.batch * 1000.0 / ms_step
    step_bytes = nums["weight_bytes"] + kv_tokens * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms_step * 1e-3) / 1e9

    # ---------------------------------------------------------------- end to end through Engine.generate
    e2e_prompts = prompts_for(args.batch)
    # long enough that the first steps after the prompts (the SM clock is still under the power cap of the prompt
    # steps: 1.15 ms per step falling to 1.02 within some fifty steps) do not set the number
    e2e_new = max(args.steps, 256)
    engine.generate(e2e_prompts, 4, greedy, stop_ids=[])          # warm the path: the same shapes, so their graphs exist
    torch.cuda.synchronize()
    # three runs, the median one is reported (the host takes part in this number: it varies more than the device's)
    runs = []
    for _ in range(3):
        t0 = time.perf_counter()
        h2d0, steps0 = engine.h2d_bytes, engine.steps_run
        results, metrics = engine.generate(e2e_prompts, e2e_new, greedy, stop_ids=[])
        torch.cuda.synchronize()
        runs.append((metrics.decode_tok_s, (engine.h2d_bytes - h2d0) / max(1, engine.steps_run - steps0),
                     time.perf_counter() - t0))
    runs.sort()
    # every step copies its positions, slots, lengths and (when they changed) page tables to the device and the
    # chosen tokens (int32 per sequence) and the status word (int32) back to the host; the prompt's token ids go up
    # with the first step
    e2e = dict(value=round(runs[1][0], 2), unit="tokens/s", h2d_bytes_per_step=round(runs[1][1]),
               d2h_bytes_per_step=4 * args.batch + 4, new_tokens=e2e_new, wall_s=round(runs[1][2], 3),
               runs=[round(r[0], 1) for r in runs])

    # ---------------------------------------------------------------- prefill of 2,048 tokens
    prompt = [rng.randrange(V) for _ in range(PREFILL_TOKENS)]

    def prefill_once():
        s = engine.acquire()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        engine.step([(s, prompt, [PREFILL_TOKENS - 1])], check=False, greedy=True)       # ends with the first token chosen
        e1.record()
        torch.cuda.synchronize()
        engine.check()
        engine.release(s)
        return e0.elapsed_time(e1)

    for _ in range(3):
        prefill_once()
    pre_ms = sorted(prefill_once() for _ in range(5))[2]
    flops = prefill_flops(cfg, PREFILL_TOKENS)
    flop_peak = peaks["bf16_tflops"] * 1e12
    if fp32:
        flop_peak = 148 * 128 * 2 * (clock_info.get("sm_max_mhz") or 1965) * 1e6
    prefill = dict(value=round(PREFILL_TOKENS / (pre_ms * 1e-3), 1), tokens=PREFILL_TOKENS, ms=round(pre_ms, 3),
                   frac=round(flops / (pre_ms * 1e-3) / flop_peak, 4))

    # ---------------------------------------------------------------- other batch sizes
    pts = {}
    for b in points:
        ms_b, _, _, _ = decode_run(b, max(8, args.steps // 2), 3)
        pts[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 1)

    # ---------------------------------------------------------------- per-phase timings, on request
    phases_out = None
    if args.profile_phases:
        from spissa_b200 import phases as ph
        engine.profile_phases = True
        engine.phase_totals.clear()
        s = engine.acquire()
        engine.step([(s, prompt, [PREFILL_TOKENS - 1])], greedy=True)
        engine.release(s)
        short = [prompts_for(args.batch)[b][:256] for b in range(args.batch)]
        slots = [engine.acquire() for _ in range(args.batch)]
        engine.step([(sl, p, []) for sl, p in zip(slots, short)], check=True)
        engine.phase_totals.pop("decode", None)
        n_dec = 4
        for i in range(n_dec):
            engine.step([(sl, [7 + i], [0]) for sl in slots], greedy=True)
        for sl in slots:
            engine.release(sl)
        engine.profile_phases = False
        L = len(engine.model.spec.schedule)
        pre = engine.phase_totals["prefill"]
        dec = engine.phase_totals["decode"]
        # the prompt entry sums the 2,048-token prompt and the short prompts that the decode steps start from
        phases_out = {"prompt_steps": dict(steps=pre["steps"], tokens=pre["tokens"], **ph.summary(dict(pre["ms"]), L)),
                      "decode_part_by_part_per_step": dict(batch=args.batch, context=256,
                                                           **ph.summary({k: v / n_dec for k, v in dec["ms"].items()}, L))}

    line = {
        "metric": "decode tokens/s (%s, batch %d, ~%d-token prompts)" % (work["model"], args.batch, PROMPT),
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32" if fp32 else "bf16", "data": "synthetic token ids, random N(0,0.02) weights", "impl": "ours",
        "config": {
            "model": work["model"], "layers": cfg.num_hidden_layers, "layers_full": full_layers,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len_mean": round(sum(prompt_lens) / len(prompt_lens)),
            "prompt_len_min": min(prompt_lens), "prompt_len_max": max(prompt_lens), "page_size": engine.page_size,
            "tied_head": bool(cfg_dict.get("tie_word_embeddings")), "decode_steps": args.steps,
            "parallelism": "single-gpu", "l2": "inputs larger than L2 (%.2f GB of weights per step)" % (nums["weight_bytes"] / 1e9),
            "peaks": peaks["source"],
        },
        "clocks": clock_info,
        "e2e": e2e,
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": pts,
    }
    if phases_out is not None:
        line["phases"] = phases_out
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
