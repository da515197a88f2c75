from __future__ import annotations

import torch

from .. import kernels
from .base import PositionEncoding, register_part


@register_part("position", "rope_half_split")
class RotaryHalfSplit(PositionEncoding):
    """Rotary encoding over the pairs (j, j + d/2): phi = p / theta^(2j/d),
    (a, b) -> (a cos phi - b sin phi, b cos phi + a sin phi)
    (xsmccc/llaisys src/ops/rope/cpu/rope_cpu.cpp:16-46, which computes the angle in double
    precision from theta held as a C float).  The cos/sin table is built once in float64 on the
    host, kept in float32, and grows with the longest position asked for.  params: head_dim, theta."""
    capturable = True


    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.head_dim = int(spec.params["head_dim"])
        self.theta = float(torch.tensor(float(spec.params["theta"]), dtype=torch.float32))
        if self.head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head size, got {self.head_dim}")
        self._cos = self._sin = None

    def table(self, positions: int):
        if self._cos is None or self._cos.shape[0] < positions:
            rows = max(positions, 2 * (self._cos.shape[0] if self._cos is not None else 0))
            half = self.head_dim // 2
            j = torch.arange(half, dtype=torch.float64)
            freq = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64), 2.0 * j / self.head_dim)
            ang = torch.arange(rows, dtype=torch.float64)[:, None] * freq[None, :]
            self._cos = torch.cos(ang).to(torch.float32).to(self.env.device)
            self._sin = torch.sin(ang).to(torch.float32).to(self.env.device)
        return self._cos, self._sin

    def fused_tables(self, positions: int):
        """(cos, sin) for kernels that apply this rotation themselves (decode attention)."""
        return self.table(positions)

    def prepare(self, max_positions):
        self.table(max_positions)          # full size once: a captured step must not see the table move

    def apply(self, qkv, num_heads, num_kv_heads, ctx, append=None):
        cos, sin = self.table(ctx.max_position + 1)
        kernels.rope_append(qkv, num_heads, num_kv_heads, self.head_dim, cos=cos, sin=sin,
                            tok_pos=ctx.tok_pos, append=append, err=ctx.err)
