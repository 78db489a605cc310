"""Grouped-query attention over the paged cache, as a mixer.

In order (src/models/qwen3/qwen3.cpp:140-179): q, k, v projections without
bias; optional RMSNorm over each head of q and k before the rotation; rotary
positions on q and k; the new keys and values go into the cache; attention
of the new queries over everything the cache holds for their sequence
(causal, optionally only the last `window` keys); output projection.  Query
head h reads key/value head h // (n_heads // n_kv_heads).

The three projections are packed into one weight at load time so that one
product makes q, k and v (upstream runs three).  All sizes, the eps of the
q/k norm, the window and the softmax scale are parameters.
"""
from __future__ import annotations

import torch

from ..cache import KVRequirement
from ..ops import kernels, linear
from ..weights.loader import TensorWant
from .base import Mixer, register_part


class GQAAttention(Mixer):
    kind = "gqa_attention"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        h, n_q, n_kv, d = (params[k] for k in ("hidden_size", "n_heads", "n_kv_heads", "head_dim"))
        w = {"q_proj": TensorWant((n_q * d, h)), "k_proj": TensorWant((n_kv * d, h)),
             "v_proj": TensorWant((n_kv * d, h)), "o_proj": TensorWant((h, n_q * d))}
        if params.get("qk_norm", False):
            w["q_norm"] = TensorWant((d,), "norm")
            w["k_norm"] = TensorWant((d,), "norm")
        return w

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.hidden = int(params["hidden_size"])
        self.n_q, self.n_kv, self.d = int(params["n_heads"]), int(params["n_kv_heads"]), int(params["head_dim"])
        if self.n_q % self.n_kv:
            raise ValueError(f"{self.n_q} query heads are no multiple of {self.n_kv} key/value heads")
        self.window = params.get("window")
        self.scale = float(params.get("softmax_scale", self.d ** -0.5))
        self.qk_norm = bool(params.get("qk_norm", False))
        self.eps = float(params.get("qk_norm_eps", 1e-6))
        q_rows, kv_rows = self.n_q * self.d, self.n_kv * self.d
        self.w_qkv = torch.empty((q_rows + 2 * kv_rows, self.hidden), dtype=load.dtype("q_proj", "k_proj", "v_proj"),
                                 device=rt.device)
        load("q_proj", out=self.w_qkv[:q_rows])
        load("k_proj", out=self.w_qkv[q_rows:q_rows + kv_rows])
        load("v_proj", out=self.w_qkv[q_rows + kv_rows:])
        self.w_o = load("o_proj")
        self.q_norm = load("q_norm") if self.qk_norm else None
        self.k_norm = load("k_norm") if self.qk_norm else None
        self._no_rotary = None

    def cache_requirement(self):
        return KVRequirement(self.n_kv, self.d, self.window)

    def step(self, x, ctx, cache, position, writes_cache=True):
        kv = cache.kv
        tables = position.rotary_tables() if position is not None else None
        if tables is None:
            if self._no_rotary is None:
                n_pos = kv.block_table.shape[1] * kv.page_size
                empty = torch.zeros((n_pos, 0), dtype=torch.float32, device=x.device)
                self._no_rotary = (empty, empty, 0)
            tables = self._no_rotary
        cos, sin, rotary_dim = tables
        qkv = linear(x, self.w_qkv)
        q = kernels.qk_norm_rope_append(qkv, self.n_q, self.n_kv, self.d, self.q_norm, self.k_norm, self.eps,
                                        cos, sin, rotary_dim, ctx.tok_pos, ctx.tok_slot, kv.k_pool, kv.v_pool,
                                        kv.block_table, ctx.status, append=writes_cache)
        o = self.attend(q, kv, ctx)
        return linear(o, self.w_o)

    def attend(self, q, kv, ctx):
        """Attention of q [n, n_q, d] over the cache; returns [n, n_q * d].

        bfloat16 with heads of 128 and pages that are a multiple of 64 tokens: the tcgen05 kernels (flash
        attention for runs of tokens, split-KV when every sequence brings one token and the group is at most
        16).  Otherwise bfloat16 with a head size the mma.sync kernels take: the split-KV kernel for single
        tokens, the flash kernel for runs.  Everything else (float32, other head sizes, larger groups in
        decode) goes to the exact-order kernel."""
        if (not ctx.all_single and ctx.q_tiles128 is not None
                and kernels.tcgen05_attention_takes(q.dtype, self.d, kv.page_size)):
            return kernels.attention_prefill_tcgen05(q, kv.k_pool, kv.v_pool, kv.block_table, ctx.q_tiles128,
                                                     self.scale, self.window or 0,
                                                     rows_covered=ctx.n_tokens == sum(ctx.seq_lens))
        if ctx.all_single and kernels.tcgen05_decode_takes(q.dtype, self.d, kv.page_size, self.n_q // self.n_kv):
            return kernels.attention_decode_tcgen05(q, kv.k_pool, kv.v_pool, kv.block_table, ctx.tok_pos, ctx.tok_slot,
                                                    self.scale, self.window or 0)
        if kernels.mma_attention_takes(q.dtype, self.d):
            if ctx.all_single and self.n_q // self.n_kv <= 16:
                return kernels.attention_decode_bf16(q, kv.k_pool, kv.v_pool, kv.block_table, ctx.tok_pos,
                                                     ctx.tok_slot, self.scale, self.window or 0)
            if not ctx.all_single and ctx.q_tiles is not None:
                return kernels.attention_prefill_bf16(q, kv.k_pool, kv.v_pool, kv.block_table, ctx.q_tiles,
                                                      self.scale, self.window or 0,
                                                      rows_covered=ctx.n_tokens == sum(ctx.seq_lens))
        return kernels.attention_generic(q, kv.k_pool, kv.v_pool, kv.block_table, ctx.tok_pos, ctx.tok_slot,
                                         self.scale, self.window or 0, ctx.status)


register_part(GQAAttention.kind, GQAAttention)
