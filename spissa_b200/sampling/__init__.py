"""Greedy and temperature / top-k / top-p sampling."""
from .sampler import Sampler, SamplingParams, draw_seed, seeded_unit, uniforms

__all__ = ["Sampler", "SamplingParams", "draw_seed", "seeded_unit", "uniforms"]
