"""Tokenizer round trips and the command line's argument handling (no GPU)."""
import json

import pytest

from spissa_b200.cli import main, render_llama3_turn
from spissa_b200.tokenizer import Tokenizer, _byte_table


def toy_tokenizer(tmp_path):
    table = _byte_table()
    vocab = {table[b]: b for b in range(256)}
    merges = []
    def add(a, b):
        merges.append(f"{a} {b}")
        vocab[a + b] = len(vocab)
    sp = table[ord(" ")]
    add("h", "e"); add("l", "l"); add("he", "ll"); add("hell", "o"); add(sp, "w"); add("o", "r")
    data = {"model": {"type": "BPE", "vocab": vocab, "merges": merges},
            "added_tokens": [{"id": 1000, "content": "<|eot_id|>"}, {"id": 1001, "content": "<|begin_of_text|>"}]}
    (tmp_path / "tokenizer.json").write_text(json.dumps(data))
    return Tokenizer(tmp_path)


def test_bpe_merges_by_rank_and_round_trips(tmp_path):
    tok = toy_tokenizer(tmp_path)
    ids = tok.encode("hello world")
    assert ids[0] == tok.vocab["hello"] and tok.vocab[_byte_table()[32] + "w"] in ids
    assert tok.decode(ids) == "hello world"
    text = "héllo wörld ∑ 123\n\n x"
    assert tok.decode(tok.encode(text)) == text


def test_special_tokens_are_matched_first(tmp_path):
    tok = toy_tokenizer(tmp_path)
    ids = tok.encode("<|begin_of_text|>hello<|eot_id|>")
    assert ids[0] == 1001 and ids[-1] == 1000 and tok.token_id("<|eot_id|>") == 1000
    assert tok.decode(ids) == "hello" and "<|eot_id|>" in tok.decode(ids, skip_special=False)


def test_missing_tokenizer_is_a_clear_error(tmp_path):
    with pytest.raises(FileNotFoundError, match="token ids"):
        Tokenizer(tmp_path)


def test_llama3_template_matches_the_reference():
    first = render_llama3_turn(False, False, " be brief ", " hi ")
    assert first.startswith("<|begin_of_text|><|start_header_id|>system<|end_header_id|>\n\nCutting Knowledge Date")
    assert "be brief<|eot_id|><|start_header_id|>user<|end_header_id|>\n\nhi<|eot_id|>" in first
    assert first.endswith("<|start_header_id|>assistant<|end_header_id|>\n\n")
    later = render_llama3_turn(True, False, None, "more")
    assert later.startswith("<|eot_id|><|start_header_id|>user")
    assert render_llama3_turn(True, True, None, "more").startswith("<|start_header_id|>user")


def test_cli_needs_a_prompt(capsys):
    with pytest.raises(SystemExit):
        main(["generate", "some_dir"])
    with pytest.raises(SystemExit):
        main(["nonsense"])
