"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration and a seed.

Matrices are drawn from N(0, std) in float32 and rounded to the storage type; norm
weights are 1, or 1 + N(0, norm_std) when ``norm_std`` > 0. Tensors are drawn in name
order from one seeded generator, so the same configuration and seed give the same
file everywhere. The reference has no such mode (its fixtures are fixed values,
crates/spissa-runtime/src/models/llama/session/tests_core.rs:148-201).
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from .safetensors_io import write_safetensors


def random_tensors(specs: list, seed: int, std: float = 0.02, norm_std: float = 0.0,
                   dtype=torch.bfloat16, device="cpu") -> dict:
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out = {}
    for s in sorted({s.name: s for s in specs}.values(), key=lambda s: s.name):
        if s.kind == "int":
            out[s.name] = torch.zeros(s.shape, dtype=torch.int32, device=device)
        elif s.init == "ones":
            t = torch.ones(s.shape, dtype=torch.float32, device=device)
            if norm_std > 0:
                t = t + norm_std * torch.randn(s.shape, generator=gen, dtype=torch.float32, device=device)
            out[s.name] = t.to(dtype)
        else:
            out[s.name] = (std * torch.randn(s.shape, generator=gen, dtype=torch.float32, device=device)).to(dtype)
    return out


def write_random_model(config, folder, seed: int = 0, std: float = 0.02, norm_std: float = 0.0,
                       dtype=torch.bfloat16) -> Path:
    """Write ``folder/config.json`` and ``folder/model.safetensors`` for ``config``."""
    from ..engine.model import Model          # late: the parts import the kernels' bindings

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    model = Model(config.to_spec())
    tensors = random_tensors(model.weight_specs(), seed, std, norm_std, dtype)
    (folder / "config.json").write_text(json.dumps(config.to_dict(), indent=2))
    write_safetensors(folder / "model.safetensors", tensors,
                      metadata={"format": "pt", "seed": seed, "std": std, "norm_std": norm_std})
    return folder
