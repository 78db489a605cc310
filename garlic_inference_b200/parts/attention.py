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

import numpy as np
import torch

from ..cache import KVRequirement
from ..ops import kernels, linear
from ..weights.loader import TensorWant
from .base import Mixer, register_part


def query_runs(shape, rows: int) -> np.ndarray:
    """The step's rows cut into runs of at most `rows` consecutive tokens of one sequence, the way the
    tensor-core prompt kernels take their queries: int32 [n_runs, 4] = {slot, first row, rows, position of the
    first row}.  The runs with the most keys to walk go first, so that the last blocks to start are short."""
    runs = [(s, st + r0, min(rows, n - r0), p + r0)
            for s, st, n, p in zip(shape.seq_slots, shape.seq_starts, shape.seq_lens, shape.seq_past)
            for r0 in range(0, n, rows)]
    runs.sort(key=lambda t: -(t[3] + t[2]))
    return np.asarray(runs, dtype=np.int32).reshape(-1, 4)


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

    def _run_rows(self, kv) -> int:
        """Height of the query runs the prompt kernel for this head size, type and page size takes (0: the
        exact-order kernel, which needs none)."""
        if kernels.tcgen05_attention_takes(self.rt.dtype, self.d, kv.page_size):
            return 128
        return 64 if kernels.mma_attention_takes(self.rt.dtype, self.d) else 0

    def step_arrays(self, shape, cache):
        rows = 0 if shape.all_single else self._run_rows(cache.kv)
        return {f"query_runs_{rows}": lambda: query_runs(shape, rows)} if rows else {}

    def _runs(self, ctx, rows: int) -> torch.Tensor:
        runs = ctx.arrays.get(f"query_runs_{rows}")
        if runs is None:                      # a context put together by hand: cut and copy here
            runs = torch.from_numpy(query_runs(ctx, rows)).to(ctx.tok_pos.device)
            ctx.arrays[f"query_runs_{rows}"] = runs
        return runs

    def attend(self, q, kv, ctx):
        """Attention of q [n, n_q, d] over the cache; returns [n, n_q * d].

        bfloat16 with heads of 128 and pages that are a multiple of 64 tokens: the tcgen05 kernels (flash
        attention for runs of tokens, split-KV when every sequence brings one token and the group is at most
        16).  Otherwise bfloat16 with a head size the mma.sync kernels take: the split-KV kernel for single
        tokens, the flash kernel for runs.  Everything else (float32, other head sizes, larger groups in
        decode) goes to the exact-order kernel."""
        covered = (not ctx.all_single) and ctx.n_tokens == sum(ctx.seq_lens)
        if ctx.all_single:
            if kernels.tcgen05_decode_takes(q.dtype, self.d, kv.page_size, self.n_q // self.n_kv):
                return kernels.attention_decode_tcgen05(q, kv.k_pool, kv.v_pool, kv.block_table, ctx.tok_pos,
                                                        ctx.tok_slot, self.scale, self.window or 0)
            if kernels.mma_attention_takes(q.dtype, self.d) and self.n_q // self.n_kv <= 16:
                return kernels.attention_decode_bf16(q, kv.k_pool, kv.v_pool, kv.block_table, ctx.tok_pos,
                                                     ctx.tok_slot, self.scale, self.window or 0)
        elif ctx.seq_lens:
            rows = self._run_rows(kv) if q.dtype == self.rt.dtype else 0
            if rows == 128:
                return kernels.attention_prefill_tcgen05(q, kv.k_pool, kv.v_pool, kv.block_table, self._runs(ctx, 128),
                                                         self.scale, self.window or 0, rows_covered=covered)
            if rows == 64:
                return kernels.attention_prefill_bf16(q, kv.k_pool, kv.v_pool, kv.block_table, self._runs(ctx, 64),
                                                      self.scale, self.window or 0, rows_covered=covered)
        return kernels.attention_generic(q, kv.k_pool, kv.v_pool, kv.block_table, ctx.tok_pos, ctx.tok_slot,
                                         self.scale, self.window or 0, ctx.status)


register_part(GQAAttention.kind, GQAAttention)
