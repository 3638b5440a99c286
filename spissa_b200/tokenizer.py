"""A byte-level BPE tokenizer read from a model folder's ``tokenizer.json``.

Only what ``--prompt`` and ``chat`` need: the Llama 3 family's scheme (split by a regular
expression, map bytes to printable characters, merge pairs by rank, special tokens matched
first). The reference ships its own byte-level BPE over the same file
(crates/spissa-runtime/src/tokenizer.rs:138-154 encode, :202-243 merges, :297-330 decode).
Token ids always work without it.
"""
from __future__ import annotations

import json
from pathlib import Path

LLAMA3_SPLIT = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|"
                r"\s*[\r\n]+|\s+(?!\S)|\s+")


def _byte_table() -> dict:
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + extra)
            extra += 1
    return table


class Tokenizer:
    def __init__(self, path):
        import regex
        path = Path(path)
        if path.is_dir():
            path = path / "tokenizer.json"
        if not path.exists():
            raise FileNotFoundError(f"no tokenizer.json at {path}; pass token ids instead of text")
        data = json.loads(path.read_text())
        model = data.get("model", {})
        if model.get("type") not in ("BPE", None):
            raise ValueError(f"tokenizer model {model.get('type')!r} is not supported (byte-level BPE only)")
        self.vocab = dict(model.get("vocab", {}))
        self.ranks = {}
        for i, m in enumerate(model.get("merges", [])):
            a, b = m.split(" ") if isinstance(m, str) else m
            self.ranks[(a, b)] = i
        self.special = {t["content"]: t["id"] for t in data.get("added_tokens", [])}
        self.id_to_token = {i: t for t, i in self.vocab.items()}
        self.id_to_token.update({i: t for t, i in self.special.items()})
        pattern = LLAMA3_SPLIT
        pre = data.get("pre_tokenizer") or {}
        for p in pre.get("pretokenizers", [pre]):
            if p.get("type") == "Split" and isinstance(p.get("pattern"), dict) and "Regex" in p["pattern"]:
                pattern = p["pattern"]["Regex"]
        self._split = regex.compile(pattern)
        self._special_split = (regex.compile("(" + "|".join(regex.escape(s) for s in
                                                            sorted(self.special, key=len, reverse=True)) + ")")
                               if self.special else None)
        self._bytes = _byte_table()
        self._unbytes = {c: b for b, c in self._bytes.items()}
        self._cache = {}

    def token_id(self, raw: str):
        return self.special.get(raw, self.vocab.get(raw))

    def _bpe(self, piece: str) -> list:
        if piece in self._cache:
            return self._cache[piece]
        parts = list(piece)
        while len(parts) > 1:
            best, where = None, -1
            for i in range(len(parts) - 1):
                r = self.ranks.get((parts[i], parts[i + 1]))
                if r is not None and (best is None or r < best):
                    best, where = r, i
            if best is None:
                break
            parts[where:where + 2] = [parts[where] + parts[where + 1]]
        ids = []
        for p in parts:
            if p not in self.vocab:
                raise ValueError(f"piece {p!r} is not in the vocabulary")
            ids.append(self.vocab[p])
        self._cache[piece] = ids
        return ids

    def encode(self, text: str) -> list:
        out = []
        chunks = self._special_split.split(text) if self._special_split else [text]
        for chunk in chunks:
            if not chunk:
                continue
            if chunk in self.special:
                out.append(self.special[chunk])
                continue
            for piece in self._split.findall(chunk):
                out.extend(self._bpe("".join(self._bytes[b] for b in piece.encode("utf-8"))))
        return out

    def decode(self, ids, skip_special: bool = True) -> str:
        buf = bytearray()
        specials = set(self.special.values())
        for i in ids:
            tok = self.id_to_token.get(int(i))
            if tok is None:
                continue
            if int(i) in specials:
                if not skip_special:
                    buf.extend(tok.encode("utf-8"))
                continue
            buf.extend(self._unbytes.get(c, ord("?")) for c in tok)
        return buf.decode("utf-8", errors="replace")
