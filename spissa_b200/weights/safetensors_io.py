"""Reading and writing the safetensors container, by tensor name.

Format: an 8-byte little-endian header length, a JSON header mapping each name to
``dtype``, ``shape`` and ``data_offsets`` (relative to the end of the header), then the
raw little-endian data (crates/spissa-import/src/safetensors.rs:261-289, :307-323).
The file is memory-mapped; a tensor is materialised only when asked for.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import torch

DTYPES = {
    "BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
    "I8": torch.int8, "I16": torch.int16, "I32": torch.int32, "I64": torch.int64, "U8": torch.uint8,
    "BOOL": torch.bool,
}
NAMES = {v: k for k, v in DTYPES.items()}
MAX_HEADER_BYTES = 100_000_000      # the reference rejects larger headers (safetensors.rs:271-274)


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One ``.safetensors`` file opened for reading by name."""

    def __init__(self, path):
        self.path = Path(path)
        if not self.path.exists():
            raise FileNotFoundError(f"no safetensors file at {self.path}")
        self._fh = open(self.path, "rb")
        head = self._fh.read(8)
        if len(head) != 8:
            raise SafetensorsError(f"{self.path}: too short for a safetensors header")
        (hlen,) = struct.unpack("<Q", head)
        if hlen > MAX_HEADER_BYTES:
            raise SafetensorsError(f"{self.path}: header length {hlen} is not plausible")
        try:
            header = json.loads(self._fh.read(hlen))
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{self.path}: header is not JSON: {e}") from None
        self.metadata = header.pop("__metadata__", {})
        self.entries = header
        self._base = 8 + hlen
        self._mm = None

    def names(self) -> list:
        return list(self.entries)

    def shape(self, name) -> tuple:
        return tuple(self.entries[name]["shape"])

    def dtype_name(self, name) -> str:
        return self.entries[name]["dtype"]

    def tensor(self, name) -> torch.Tensor:
        """A CPU tensor that owns its memory."""
        if name not in self.entries:
            raise SafetensorsError(f"{self.path}: no tensor named {name!r}")
        meta = self.entries[name]
        if meta["dtype"] not in DTYPES:
            raise SafetensorsError(f"{self.path}: tensor {name!r} has unsupported dtype {meta['dtype']}")
        dt = DTYPES[meta["dtype"]]
        lo, hi = meta["data_offsets"]
        n = 1
        for s in meta["shape"]:
            n *= s
        if n * torch.empty((), dtype=dt).element_size() != hi - lo:
            raise SafetensorsError(f"{self.path}: tensor {name!r} has {hi - lo} bytes, its shape wants "
                                   f"{n * torch.empty((), dtype=dt).element_size()}")
        if n == 0:
            return torch.empty(meta["shape"], dtype=dt)
        if self._mm is None:
            self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        buf = memoryview(self._mm)[self._base + lo:self._base + hi]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")          # read-only buffer: we clone at once
            t = torch.frombuffer(buf, dtype=dt, count=n)
        return t.reshape(meta["shape"]).clone()

    def close(self):
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:
                pass
            self._mm = None
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def write_safetensors(path, tensors: dict, metadata: dict | None = None) -> None:
    """Write ``tensors`` (name → CPU tensor) in name order."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} of tensor {name!r}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                flat = t.reshape(-1)
                flat = flat.to(torch.uint8) if t.dtype == torch.bool else flat.view(torch.uint8)
                fh.write(flat.numpy().tobytes())
