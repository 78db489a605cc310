"""Arrangements of a layer's parts, and the two ends of the model.

`pre_norm_residual` (src/models/qwen3/qwen3.cpp:225-248):
    r = h;  x = norm_in(h);  r = mixer(x) + r;  x = norm_post(r);  h = ffn(x) + r
The residual stream is float32; each add happens inside the norm that
follows it, so the block takes and returns a pending `delta` (see base.py).
"""
from __future__ import annotations

import torch

from ..ops import kernels, linear
from ..weights.loader import TensorWant
from .base import Block, Embedding, Head, register_part


class PreNormResidualBlock(Block):
    kind = "pre_norm_residual"
    norm_names = ("input", "post_mixer")

    def __init__(self, mixer, feed_forward, norms, position, rt):
        self.rt = rt
        self.mixer, self.feed_forward, self.position = mixer, feed_forward, position
        missing = [n for n in self.norm_names if n not in norms]
        if missing:
            raise ValueError(f"block 'pre_norm_residual' needs norms {self.norm_names}; missing {missing}")
        self.norm_in, self.norm_post = norms["input"], norms["post_mixer"]

    def cache_requirement(self):
        return self.mixer.cache_requirement()

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in (self.mixer, self.feed_forward, self.norm_in, self.norm_post)) and \
            (self.position is None or self.position.graph_safe)

    def step_arrays(self, shape, cache):
        return {**self.mixer.step_arrays(shape, cache), **self.feed_forward.step_arrays(shape, cache)}

    def step(self, delta, residual, ctx, cache, writes_cache=True):
        x = self.norm_in.add_norm(delta, residual)
        a = self.mixer.step(x, ctx, cache, self.position, writes_cache)
        x = self.norm_post.add_norm(a, residual)
        return self.feed_forward.step(x, ctx)


class TokenEmbedding(Embedding):
    """h[t] = table[id[t]], no scaling (src/src-cuda/embedding.cu:29-53), written as float32."""
    kind = "token_embedding"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        return {"weight": TensorWant((params["vocab_size"], params["hidden_size"]), "table")}

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.weight = load("weight")

    def step(self, ctx):
        return kernels.embedding(ctx.tokens, self.weight)


class LinearHead(Head):
    """logits = normed . W^T as float32 (src/models/qwen3/qwen3.cpp:302-303), on the rows asked for only."""
    kind = "linear_head"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        return {"weight": TensorWant((params["vocab_size"], params["hidden_size"]), "table")}

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.weight = load("weight")

    def step(self, normed):
        return linear(normed, self.weight, out_dtype=torch.float32)


register_part(PreNormResidualBlock.kind, PreNormResidualBlock)
register_part(TokenEmbedding.kind, TokenEmbedding)
register_part(LinearHead.kind, LinearHead)
