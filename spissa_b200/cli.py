"""Command line in the manner of the reference's ``spissa`` binary.

    python -m spissa_b200 generate MODEL_DIR --token-ids 1,2,3 [--token-ids 4,5] --max-new-tokens 16
    python -m spissa_b200 generate --random CONFIG.json --seed 1 --token-ids 1,2,3
    python -m spissa_b200 chat MODEL_DIR --temp 0.6 --top-p 0.95

Option names and meanings follow ``spissa chat`` (crates/spissa-cli/src/main.rs:271-327):
``--ctx`` cache cap in tokens (default 2048), ``--max-new-tokens`` (chat 512), ``--temp`` (0 =
greedy), ``--top-p`` (0.95, used when --temp > 0), ``--top-k`` (0 = no cap), ``--seed`` (0),
``--chat-template`` (llama3 | raw), ``--system``; ``--token-ids`` and ``--logits-out`` as in
``spissa run`` (main.rs:133-195). ``--repeat-penalty`` exists in the reference for its Qwen
chat only and is not offered here.
"""
from __future__ import annotations

import argparse
import json
import sys
import tempfile


def _sampling_args(p, max_new_default):
    p.add_argument("--ctx", type=int, default=2048, help="context length: tokens the cache holds per sequence")
    p.add_argument("--max-new-tokens", type=int, default=max_new_default)
    p.add_argument("--temp", type=float, default=0.0, help="sampling temperature; 0 = greedy")
    p.add_argument("--top-p", type=float, default=0.95, dest="top_p", help="nucleus cutoff, used when --temp > 0")
    p.add_argument("--top-k", type=int, default=0, dest="top_k", help="keep the K most probable tokens (0 = no cap)")
    p.add_argument("--seed", type=int, default=0, help="seed of the sampling draws")
    p.add_argument("--dtype", default="bf16", choices=["bf16", "fp32", "bfloat16", "float32"])
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--profile-phases", action="store_true", dest="profile_phases",
                   help="time every phase of the block with CUDA events (steps then run kernel by kernel, part by part) "
                        "and print the sums, as the reference's llama-test --profile-phases does")


def _engine(args, n_seqs):
    from . import Engine, load_config, write_random_model
    max_tokens = ((args.ctx + 63) // 64 * 64) * max(1, n_seqs)
    if getattr(args, "random", None):
        cfg = load_config(args.random)
        folder = tempfile.mkdtemp(prefix="spissa_b200_random_")
        write_random_model(cfg, folder, seed=args.weights_seed)
        return Engine.from_folder(folder, dtype=args.dtype, max_tokens=max_tokens, max_seqs=max(1, n_seqs),
                                  device=args.device)
    if not args.model:
        raise SystemExit("give a model folder or --random CONFIG.json")
    return Engine.from_folder(args.model, dtype=args.dtype, max_tokens=max_tokens, max_seqs=max(1, n_seqs),
                              device=args.device)


def _phase_report(engine) -> dict:
    """Per kind of step (prefill, decode): steps, tokens and the phases' milliseconds summed over the run."""
    from . import phases
    out = {}
    for kind, acc in engine.phase_totals.items():
        out[kind] = dict(steps=acc["steps"], tokens=acc["tokens"],
                         **phases.summary(acc["ms"], len(engine.model.spec.schedule)))
    return out


def cmd_generate(args) -> int:
    from . import SamplingParams
    prompts = [[int(x) for x in ids.split(",") if x.strip()] for ids in (args.token_ids or [])]
    tok = None
    if args.prompt:
        from .tokenizer import Tokenizer
        tok = Tokenizer(args.model)
        prompts += [tok.encode(p) for p in args.prompt]
    if not prompts:
        raise SystemExit("give --token-ids a,b,c (repeatable) or --prompt TEXT")
    engine = _engine(args, len(prompts))
    engine.profile_phases = bool(args.profile_phases)
    params = SamplingParams(args.temp, args.top_k, args.top_p, args.seed)
    stop = [int(x) for x in args.stop_ids.split(",")] if args.stop_ids else None
    results, m = engine.generate(prompts, args.max_new_tokens, params, stop_ids=stop,
                                 return_logits=bool(args.logits_out))
    for r in results:
        line = {"request": r.request, "prompt_tokens": r.prompt_tokens, "tokens": r.tokens,
                "finish_reason": r.finish_reason}
        if tok is not None:
            line["text"] = tok.decode(r.tokens)
        print(json.dumps(line))
    print(json.dumps({"ttft_ms": round(m.ttft_ms, 3), "prefill_ms": round(m.prefill_ms, 3),
                      "decode_ms": round(m.decode_ms, 3), "decode_tok_s": round(m.decode_tok_s, 2),
                      "batches": m.batches, "steps": m.steps}), file=sys.stderr)
    if args.profile_phases:
        print(json.dumps({"phases": _phase_report(engine)}), file=sys.stderr)
    if args.logits_out:
        # the first step's logits of every request, like the reference's --logits-out
        with open(args.logits_out, "w") as fh:
            json.dump({"first_step_logits": [r.logits[0].tolist() for r in results]}, fh)
    return 0


def render_llama3_turn(has_context, previous_ended, system, text) -> str:
    """The Llama 3 template of the reference (crates/spissa-cli/src/chat_template.rs:138-163)."""
    out = ""
    if not has_context:
        out += "<|begin_of_text|><|start_header_id|>system<|end_header_id|>\n\n"
        out += "Cutting Knowledge Date: December 2023\nToday Date: 26 Jul 2024\n\n"
        if system and system.strip():
            out += system.strip()
        out += "<|eot_id|>"
    elif not previous_ended:
        out += "<|eot_id|>"
    out += "<|start_header_id|>user<|end_header_id|>\n\n" + text.strip() + "<|eot_id|>"
    out += "<|start_header_id|>assistant<|end_header_id|>\n\n"
    return out


def cmd_chat(args) -> int:
    from . import SamplingParams
    from .engine.session import ChatSession
    from .tokenizer import Tokenizer
    tok = Tokenizer(args.model)
    engine = _engine(args, 1)
    engine.profile_phases = bool(args.profile_phases)
    session = ChatSession(engine, SamplingParams(args.temp, args.top_k, args.top_p, args.seed), max_seq_len=args.ctx)
    stop = set(engine.config.stop_token_ids())
    if args.chat_template == "llama3":
        for raw in ("<|eot_id|>", "<|end_of_text|>"):           # chat_template.rs:89-112
            if tok.token_id(raw) is not None:
                stop.add(tok.token_id(raw))
    has_context, ended = False, False
    print("type 'exit' to leave", file=sys.stderr)
    while True:
        try:
            text = input("you> ").strip()
        except EOFError:
            break
        if text in ("exit", "quit", "/exit", "/quit"):
            break
        if not text:
            continue
        turn = (render_llama3_turn(has_context, ended, args.system, text) if args.chat_template == "llama3"
                else ("\n" + text if has_context else text))
        reply = []
        sys.stdout.write("bot> ")

        def on_token(t):
            if t in stop:
                return False
            reply.append(t)
            return True

        res = session.generate_turn(tok.encode(turn), args.max_new_tokens, on_token)
        print(tok.decode(reply))
        ended = res.finish_reason == "stop"
        has_context = True
        print(f"  [{len(res.tokens)} tok, {res.decode_tok_s:.1f} tok/s, ctx {res.context_len}]", file=sys.stderr)
        if args.profile_phases:
            print("  " + json.dumps({"phases": _phase_report(engine)}), file=sys.stderr)
            engine.phase_totals.clear()
    session.close()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="spissa_b200", description="Llama generation on one B200")
    sub = ap.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="generate for one or more prompts given as token ids (or text)")
    g.add_argument("model", nargs="?", help="folder with config.json and model.safetensors")
    g.add_argument("--random", metavar="CONFIG.json", help="random weights for this configuration instead of a folder")
    g.add_argument("--weights-seed", type=int, default=0)
    g.add_argument("--token-ids", action="append", help="comma-separated token ids; repeat for a batch")
    g.add_argument("--prompt", action="append", help="text; needs tokenizer.json in the model folder")
    g.add_argument("--stop-ids", help="comma-separated stop token ids (default: the configuration's eos)")
    g.add_argument("--logits-out", help="write the first step's logits as JSON")
    _sampling_args(g, 64)
    g.set_defaults(fn=cmd_generate)
    c = sub.add_parser("chat", help="interactive multi-turn chat (needs tokenizer.json)")
    c.add_argument("model")
    c.add_argument("--chat-template", default="llama3", choices=["llama3", "raw"])
    c.add_argument("--system", default=None)
    _sampling_args(c, 512)
    c.set_defaults(fn=cmd_chat)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
