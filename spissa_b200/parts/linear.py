"""y = x · Wᵀ with W stored [out, in] (crates/spissa-runtime/src/ops.rs:62-105).

``Linear`` holds one weight matrix and picks the kernel for a call by the operands'
storage types and sizes: bfloat16 activations on a bfloat16 weight go to the weight-streaming
kernel for a few tokens (decoding), to the tcgen05 kernel that streams the weight with its rows as the
instruction's M for a few dozen tokens, and to the tcgen05 tile kernel otherwise, when the rows are
multiples of 16 bytes; everything else, and the whole 32-bit path, goes to the FFMA kernel.
"""
from __future__ import annotations

import torch

from ..csrc import lib as K

_SM_COUNT: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of ``device`` (the current CUDA device when None), asked once per device."""
    index = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    if index not in _SM_COUNT:
        _SM_COUNT[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return _SM_COUNT[index]
GEMV_TOKENS = 16          # up to this many tokens the weight-streaming kernel runs instead of 128-row tiles
GATED_GEMV_TOKENS = 16    # the same for the gate/up product
STREAM_TOKENS = 64        # from there up to this many tokens the weight streams through tcgen05 with the tokens as the
#                           instruction's N (at 64 tokens: QKV 9.4 vs 12.8 us, gate/up 29 vs 40 us, down 14.4 vs 19.5 us)


def tile_width(M: int, N: int, sms: int | None = None) -> int:
    """256-wide tiles (half the shared-memory traffic per FLOP) when they still occupy most SMs, else 128-wide;
    192-wide when that saves a round of tiles: 2,048 tokens x 3,072 outputs are 192 tiles of 256 columns, two
    rounds on 148 SMs of which the second is a third full, but 256 tiles of 192 columns, two rounds of shorter tiles."""
    SM_COUNT = sms if sms else sm_count()
    m_tiles = (M + 127) // 128
    tiles_256 = m_tiles * ((N + 255) // 256)
    if tiles_256 < (SM_COUNT * 2) // 3:
        return 128
    if M > 128:
        cost_256 = -(-tiles_256 // SM_COUNT) * 256
        cost_192 = -(-(m_tiles * ((N + 191) // 192)) // SM_COUNT) * 192
        if cost_192 * 10 <= cost_256 * 9:
            return 192
    return 256


class Linear:
    def __init__(self, weight: torch.Tensor):
        if weight.dim() != 2:
            raise ValueError("a linear weight is a matrix [out, in]")
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape

    def __call__(self, x: torch.Tensor, out: torch.Tensor | None = None, out_dtype=None,
                 accumulate: bool = False) -> torch.Tensor:
        """``accumulate`` adds the product into ``out`` (float32) instead of overwriting it."""
        if out is None:
            if accumulate:
                raise ValueError("accumulation needs the tensor to add into")
            out = torch.empty(x.shape[0], self.out_features, dtype=out_dtype or x.dtype, device=x.device)
        mode = K.TC_ACCUMULATE if accumulate else K.TC_STORE
        if x.shape[0] <= GEMV_TOKENS and K.gemv_supported(x, self.weight):
            K.gemv(x, self.weight, out, mode)
        elif x.shape[0] <= STREAM_TOKENS and K.tc_stream_supported(x, self.weight, mode):
            K.tc_stream(x, self.weight, out, mode)
        elif K.tc_gemm_supported(x, self.weight):
            K.tc_gemm(x, self.weight, out, mode, tile_width(x.shape[0], self.out_features, sm_count(x.device)))
        else:
            K.gemm_generic(x, self.weight, out, accumulate=accumulate)
        return out


class GatedLinear:
    """silu(x·Wgᵀ) ⊙ (x·Wuᵀ) as one product over the stacked weight.

    When the sizes allow, gate and up rows are interleaved in blocks (``block`` gate rows, then
    the ``block`` up rows of the same outputs) so that one tile of the tensor-core kernel holds
    both halves and applies silu·up in its epilogue.
    """

    def __init__(self, gate: torch.Tensor, up: torch.Tensor):
        I = gate.shape[0]
        self.intermediate = I
        self.block = 128 if I % 128 == 0 else 64 if I % 64 == 0 else 0
        fused = self.block and gate.dtype == torch.bfloat16 and gate.shape[1] % 8 == 0
        if fused:
            h = self.block
            g = gate.reshape(I // h, h, -1)
            u = up.reshape(I // h, h, -1)
            self.weight = torch.stack([g, u], dim=1).reshape(2 * I, -1).contiguous()
        else:
            self.block = 0
            self.weight = torch.cat([gate, up], dim=0).contiguous()
        self.plain = Linear(self.weight)

    def __call__(self, x: torch.Tensor, act_dtype) -> torch.Tensor:
        out = torch.empty(x.shape[0], self.intermediate, dtype=act_dtype, device=x.device)
        if self.block and x.shape[0] <= GATED_GEMV_TOKENS and K.gemv_supported(x, self.weight):
            K.gemv(x, self.weight, out, K.TC_SILU_MUL, self.block)
        elif self.block and x.shape[0] <= STREAM_TOKENS and K.tc_stream_supported(x, self.weight, K.TC_SILU_MUL, self.block):
            K.tc_stream(x, self.weight, out, K.TC_SILU_MUL, self.block)
        elif self.block and K.tc_gemm_supported(x, self.weight):
            K.tc_gemm(x, self.weight, out, K.TC_SILU_MUL, 2 * self.block)
        else:
            gu = self.plain(x, out_dtype=act_dtype)
            K.silu_mul(gu, out)
        return out
