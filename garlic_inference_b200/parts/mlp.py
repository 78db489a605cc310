"""SwiGLU feed-forward: down( silu(gate(x)) * up(x) ), no biases
(src/models/qwen3/qwen3.cpp:186-203).  gate and up are packed into one weight
at load time (one product instead of two); silu and the product are one kernel
in float32 with a single rounding (upstream rounds after silu and again after
the product, src/src-cuda/activations/silu.cu:35-67, hadamard.cu:48-67)."""
from __future__ import annotations

import torch

from ..ops import linear, swiglu_product
from ..weights.loader import TensorWant
from .base import FeedForward, register_part


class SwiGLUMLP(FeedForward):
    kind = "swiglu_mlp"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        h, i = params["hidden_size"], params["intermediate_size"]
        return {"gate_proj": TensorWant((i, h)), "up_proj": TensorWant((i, h)), "down_proj": TensorWant((h, i))}

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        self.w_gate_up = torch.empty((2 * self.inter, self.hidden), dtype=load.dtype("gate_proj", "up_proj"),
                                     device=rt.device)
        load("gate_proj", out=self.w_gate_up[:self.inter])
        load("up_proj", out=self.w_gate_up[self.inter:])
        self.w_down = load("down_proj")

    def step(self, x, ctx):
        return linear(swiglu_product(x, self.w_gate_up), self.w_down)


register_part(SwiGLUMLP.kind, SwiGLUMLP)
