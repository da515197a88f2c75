from __future__ import annotations

import torch

from .. import kernels
from .base import PositionEncoding, register_part

# (head_dim, theta, device) -> (cos, sin): every layer of a model has a part of its own, and all
# of them rotate by the same angles, so they share one pair of tables.
_TABLES = {}


def _tables(head_dim: int, theta: float, device, rows: int):
    key = (head_dim, theta, str(device))
    have = _TABLES.get(key)
    if have is None or have[0].shape[0] < rows:
        half = head_dim // 2
        j = torch.arange(half, dtype=torch.float64)
        freq = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float64), 2.0 * j / head_dim)
        ang = torch.arange(rows, dtype=torch.float64)[:, None] * freq[None, :]
        have = (torch.cos(ang).to(torch.float32).to(device), torch.sin(ang).to(torch.float32).to(device))
        _TABLES[key] = have
    return have


@register_part("position", "rope_half_split")
class RotaryHalfSplit(PositionEncoding):
    """Rotary encoding over the pairs (j, j + d/2): phi = p / theta^(2j/d),
    (a, b) -> (a cos phi - b sin phi, b cos phi + a sin phi)
    (xsmccc/llaisys src/ops/rope/cpu/rope_cpu.cpp:16-46, which computes the angle in double
    precision from theta held as a C float).  The cos/sin table is built in float64 on the host
    and kept in float32.  prepare() sizes it once for the longest sequence the engine can hold;
    after that it never moves (a captured step has its address), and a position beyond it is an
    error.  A part that was never prepared grows its table on demand.  params: head_dim, theta."""
    capturable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.head_dim = int(spec.params["head_dim"])
        self.theta = float(torch.tensor(float(spec.params["theta"]), dtype=torch.float32))
        if self.head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head size, got {self.head_dim}")
        self._cos = self._sin = None
        self._prepared = False

    def table(self, positions: int):
        if self._cos is None or self._cos.shape[0] < positions:
            if self._prepared:
                raise ValueError(f"position {positions - 1} lies beyond the {self._cos.shape[0]} positions the "
                                 f"rotary table was prepared for")
            rows = max(positions, 2 * (self._cos.shape[0] if self._cos is not None else 0))
            self._cos, self._sin = _tables(self.head_dim, self.theta, self.env.device, rows)
        return self._cos, self._sin

    def prepare(self, max_positions):
        self._prepared = False
        self.table(max_positions)
        self._prepared = True

    def rotation_tables(self, positions: int):
        return self.table(positions)

    def apply(self, qkv, num_heads, num_kv_heads, ctx):
        cos, sin = self.table(ctx.max_position + 1)
        kernels.rope_append(qkv, num_heads, num_kv_heads, self.head_dim, cos=cos, sin=sin,
                            tok_pos=ctx.tok_pos, err=ctx.err)
