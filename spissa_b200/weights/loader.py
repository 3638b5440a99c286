"""Weights from a model folder, by tensor name, checked against what the model expects.

The model's parts list the tensors they want (name, shape, float or integer). The
folder's ``model.safetensors`` (or the shards named by ``model.safetensors.index.json``,
crates/spissa-cli/src/commands/pack.rs:197-214) is compared with that list first; any
difference — tensors missing, tensors nobody asked for, wrong shapes, unusable
dtypes — raises ONE ``WeightError`` that lists them all
(the reference names the offending tensor: crates/spissa-runtime/src/models/llama/session/validation.rs:46-60).

Storage: floating tensors stay bfloat16; float16 is converted to bfloat16; a tensor
stored in 32-bit stays 32-bit; integer tables become int32. In the true 32-bit mode
every floating tensor is widened to float32, which is exact for bfloat16
(crates/spissa-runtime/src/tensor.rs:217-221).
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from .safetensors_io import DTYPES, SafetensorsError, SafetensorsFile

_FLOAT = {"BF16", "F16", "F32"}
_INT = {"I8", "I16", "I32", "I64", "U8"}


class WeightError(ValueError):
    """The checkpoint does not fit the model; ``missing``, ``unexpected``, ``mismatched`` say how."""

    def __init__(self, source, missing, unexpected, mismatched):
        self.missing, self.unexpected, self.mismatched = list(missing), list(unexpected), list(mismatched)
        lines = [f"weights in {source} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.mismatched:
            lines.append(f"  wrong shape or dtype ({len(self.mismatched)}): " + "; ".join(self.mismatched))
        super().__init__("\n".join(lines))


class TensorSource:
    """All tensors of a folder, a single file or a shard index, by name."""

    def __init__(self, path):
        p = Path(path)
        self.where = str(p)
        self.files = []
        self.owner = {}
        if p.is_dir():
            index = p / "model.safetensors.index.json"
            single = p / "model.safetensors"
            if index.exists():
                self._open_index(index)
            elif single.exists():
                self._open_file(single)
            else:
                raise FileNotFoundError(f"{p} holds neither model.safetensors nor model.safetensors.index.json")
        elif p.name.endswith(".index.json"):
            self._open_index(p)
        else:
            self._open_file(p)

    def _open_file(self, path):
        f = SafetensorsFile(path)
        self.files.append(f)
        for n in f.names():
            self.owner[n] = f

    def _open_index(self, path):
        idx = json.loads(Path(path).read_text())
        shards = {}
        for name, shard in idx.get("weight_map", {}).items():
            if shard not in shards:
                shards[shard] = SafetensorsFile(Path(path).parent / shard)
                self.files.append(shards[shard])
            if name not in shards[shard].entries:
                raise SafetensorsError(f"{path}: {name!r} is mapped to {shard}, which does not hold it")
            self.owner[name] = shards[shard]

    def names(self):
        return list(self.owner)

    def shape(self, name):
        return self.owner[name].shape(name)

    def dtype_name(self, name):
        return self.owner[name].dtype_name(name)

    def tensor(self, name):
        return self.owner[name].tensor(name)

    def close(self):
        for f in self.files:
            f.close()


def check_against(source: TensorSource, specs: list) -> None:
    """Raise ``WeightError`` unless ``source`` holds exactly the tensors of ``specs``."""
    want = {}
    for s in specs:
        if s.name in want and tuple(want[s.name].shape) != tuple(s.shape):
            raise ValueError(f"two parts ask for {s.name!r} with different shapes")
        want[s.name] = s
    have = set(source.names())
    missing = sorted(n for n in want if n not in have)
    unexpected = sorted(n for n in have if n not in want)
    mismatched = []
    for n in sorted(want):
        if n not in have:
            continue
        s = want[n]
        shape, dt = source.shape(n), source.dtype_name(n)
        if tuple(shape) != tuple(s.shape):
            mismatched.append(f"{n}: file has {list(shape)}, model wants {list(s.shape)}")
        elif s.kind == "float" and dt not in _FLOAT:
            mismatched.append(f"{n}: stored as {dt}, a floating tensor (BF16, F16, F32) is wanted")
        elif s.kind == "int" and dt not in _INT:
            mismatched.append(f"{n}: stored as {dt}, an integer table is wanted")
    if missing or unexpected or mismatched:
        raise WeightError(source.where, missing, unexpected, mismatched)


def storage_dtype(file_dtype: str, kind: str, full_precision: bool) -> torch.dtype:
    if kind == "int":
        return torch.int32
    if full_precision or file_dtype == "F32":
        return torch.float32
    return torch.bfloat16


def load_tensors(path, specs: list, device, full_precision: bool) -> dict:
    """name -> tensor on ``device`` in its storage dtype, after the whole-checkpoint check."""
    source = TensorSource(path)
    try:
        check_against(source, specs)
        out = {}
        for s in specs:
            if s.name in out:
                continue
            t = source.tensor(s.name)
            out[s.name] = t.to(storage_dtype(source.dtype_name(s.name), s.kind, full_precision)).to(device)
        return out
    finally:
        source.close()
