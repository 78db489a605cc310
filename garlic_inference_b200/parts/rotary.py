"""Rotary position encoding: the table of angles.

inv_freq[i] = theta^(-2i/r) for i < r/2 and angle = position * inv_freq[i],
scaling 1.0, no rope scaling (src/src-cuda/rope.cu:3-23,41-79; upstream uses
the fast `__powf`/`__sincosf`, which lose accuracy at large positions).  The
table is made once on the host in float64 and stored as float32 cos and sin
[max_positions, r/2]; the mixer's kernel does the rotation.  `rotary_dim` r
may be smaller than the head (the rest of the head passes through).
"""
from __future__ import annotations

import torch

from .base import PositionEncoding, register_part


class RotaryPositions(PositionEncoding):
    kind = "rotary"
    graph_safe = True

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        self.theta = float(params["theta"])
        self.max_positions = int(params["max_positions"])
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        cos, sin = self.build_tables(self.rotary_dim, self.theta, self.max_positions)
        self.cos = cos.to(rt.device)
        self.sin = sin.to(rt.device)

    @staticmethod
    def build_tables(rotary_dim: int, theta: float, max_positions: int):
        i = torch.arange(rotary_dim // 2, dtype=torch.float64)
        inv_freq = theta ** (-2.0 * i / rotary_dim)
        ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
        return ang.cos().to(torch.float32).contiguous(), ang.sin().to(torch.float32).contiguous()

    def rotary_tables(self):
        return self.cos, self.sin, self.rotary_dim


register_part(RotaryPositions.kind, RotaryPositions)
