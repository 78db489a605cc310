"""Python faces of the CUDA entry points.

Each function checks that its tensors are on the GPU, dense and of the types
the kernel is written for, allocates the output, and launches on torch's
current stream.  Sizes a kernel cannot take come back as `KernelError` with
the kernel's own message.
"""
from __future__ import annotations

from typing import Optional

import torch

from .library import KernelError, check, counters, require_gpu
from .library import counters as counters_mod

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


def code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is neither float32 nor bfloat16") from None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dense(t: torch.Tensor, name: str, dtype=None) -> torch.Tensor:
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; the kernels run on the GPU only")
    if not t.is_contiguous():
        raise KernelError(f"{name} of shape {tuple(t.shape)} and strides {t.stride()} is not dense")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} is {t.dtype}, the kernel wants {dtype}")
    return t


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def set_dependent_launch(on: bool) -> None:
    """Whether the launches that follow carry the attribute for programmatic dependent launch (the next
    kernel may be launched, and fetch its weights, while this one still runs)."""
    require_gpu().gi_set_pdl(1 if on else 0)


def embedding(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 rows of `table` for int32 `ids`: the start of the residual stream."""
    l = require_gpu()
    _dense(ids, "ids", torch.int32)
    _dense(table, "table")
    n, (vocab, hidden) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    _dense(out, "out", torch.float32)
    check(l.gi_embedding(_ptr(ids), _ptr(table), code(table.dtype), _ptr(out), n, vocab, hidden, _stream()), l)
    return out


def add_rmsnorm(delta: Optional[torch.Tensor], residual: torch.Tensor, weight: torch.Tensor, eps: float,
                act_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                write_residual: bool = True, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """normed = rmsnorm(residual (+ delta)) * weight in `act_dtype`; with `write_residual` the
    float32 sum goes back into `residual`.  `rows` (int32) picks input rows (then nothing is written back)."""
    l = require_gpu()
    _dense(residual, "residual", torch.float32)
    _dense(weight, "weight")
    dim = residual.shape[-1]
    if weight.numel() != dim:
        raise KernelError(f"norm weight has {weight.numel()} elements for rows of {dim}")
    if delta is not None:
        _dense(delta, "delta", act_dtype)
        if delta.shape != residual.shape:
            raise KernelError(f"delta {tuple(delta.shape)} and residual {tuple(residual.shape)} differ")
    if rows is not None:
        _dense(rows, "rows", torch.int32)
        n_rows, write_residual = rows.numel(), False
    else:
        n_rows = residual.numel() // dim
    if out is None:
        out = torch.empty((n_rows, dim), dtype=act_dtype, device=residual.device)
    _dense(out, "out", act_dtype)
    check(l.gi_add_rmsnorm(_ptr(delta), _ptr(residual), _ptr(weight), code(weight.dtype), _ptr(out),
                           code(act_dtype), _ptr(rows), n_rows, dim, float(eps), int(write_residual), _stream()), l)
    return out


def residual_add(delta: torch.Tensor, residual: torch.Tensor) -> None:
    l = require_gpu()
    _dense(delta, "delta")
    _dense(residual, "residual", torch.float32)
    if delta.shape != residual.shape:
        raise KernelError(f"delta {tuple(delta.shape)} and residual {tuple(residual.shape)} differ")
    check(l.gi_residual_add(_ptr(delta), code(delta.dtype), _ptr(residual), residual.numel(), _stream()), l)


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(gate) * up for [n, 2*inter] rows holding the gate first, then up."""
    l = require_gpu()
    _dense(gate_up, "gate_up")
    n, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError(f"gate_up rows of {two_i} columns cannot hold a gate and an up half")
    if out is None:
        out = torch.empty((n, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    _dense(out, "out", gate_up.dtype)
    check(l.gi_swiglu(_ptr(gate_up), _ptr(out), code(gate_up.dtype), n, two_i // 2, _stream()), l)
    return out


def cast(src: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if src.dtype == dtype:
        return src
    l = require_gpu()
    _dense(src, "src")
    out = torch.empty(src.shape, dtype=dtype, device=src.device)
    check(l.gi_cast(_ptr(src), code(src.dtype), _ptr(out), code(dtype), src.numel(), _stream()), l)
    return out


def random_normal(out: torch.Tensor, key: int, mean: float, std: float) -> torch.Tensor:
    """Fill `out` (float32 or bfloat16, dense) with mean + std * z_i, z_i a standard normal variate that
    depends on (key, i) alone; `weights/random_init.py` holds the same arithmetic for the host."""
    l = require_gpu()
    _dense(out, "out")
    check(l.gi_random_normal(_ptr(out), code(out.dtype), out.numel(), key & 0xFFFFFFFFFFFFFFFF, float(mean),
                             float(std), _stream()), l)
    return out


def qk_norm_rope_append(qkv: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                        q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                        cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int,
                        tok_pos: torch.Tensor, tok_slot: torch.Tensor,
                        k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                        status: torch.Tensor, append: bool = True) -> torch.Tensor:
    """Norm and rotate q and k of packed projections [n, (n_q + 2 n_kv) d]; returns q [n, n_q, d]
    and (with `append`) writes k and v of every token with a slot into the paged pools."""
    l = require_gpu()
    act = qkv.dtype
    _dense(qkv, "qkv")
    n = qkv.shape[0]
    if qkv.shape[1] != (n_q + 2 * n_kv) * head_dim:
        raise KernelError(f"qkv rows have {qkv.shape[1]} columns, not (n_q + 2 n_kv) * head_dim = "
                          f"{(n_q + 2 * n_kv) * head_dim}")
    for t, name in ((k_pool, "k_pool"), (v_pool, "v_pool")):
        _dense(t, name, act)
    n_pages, pool_kv, page_size, pool_d = k_pool.shape
    if (pool_kv, pool_d) != (n_kv, head_dim) or v_pool.shape != k_pool.shape:
        raise KernelError(f"cache pools {tuple(k_pool.shape)} / {tuple(v_pool.shape)} do not fit "
                          f"{n_kv} key/value heads of {head_dim}")
    _dense(cos, "cos", torch.float32), _dense(sin, "sin", torch.float32)
    if cos.shape != sin.shape or cos.shape[1] * 2 != rotary_dim:
        raise KernelError(f"rotary tables {tuple(cos.shape)} do not fit rotary_dim {rotary_dim}")
    for t, name in ((tok_pos, "tok_pos"), (tok_slot, "tok_slot"), (block_table, "block_table"), (status, "status")):
        _dense(t, name, torch.int32)
    if tok_pos.numel() < n or tok_slot.numel() < n:
        raise KernelError("tok_pos / tok_slot are shorter than the token rows")
    w_code = F32
    if q_weight is not None:
        _dense(q_weight, "q_weight"), _dense(k_weight, "k_weight", q_weight.dtype)
        if q_weight.numel() != head_dim or k_weight.numel() != head_dim:
            raise KernelError("q/k norm weights must have head_dim elements")
        w_code = code(q_weight.dtype)
    q_out = torch.empty((n, n_q, head_dim), dtype=act, device=qkv.device)
    check(l.gi_qk_norm_rope_append(
        _ptr(qkv), _ptr(q_out), _ptr(k_pool), _ptr(v_pool), code(act), _ptr(q_weight), _ptr(k_weight), w_code,
        float(eps), _ptr(cos), _ptr(sin), rotary_dim, _ptr(tok_pos), _ptr(tok_slot), _ptr(block_table),
        n, n_q, n_kv, head_dim, page_size, block_table.shape[1], n_pages, cos.shape[0], int(append),
        _ptr(status), _stream()), l)
    return q_out


def attention_generic(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                      tok_pos: torch.Tensor, tok_slot: torch.Tensor, scale: float, window: int,
                      status: torch.Tensor) -> torch.Tensor:
    """Exact-order attention of q [n, n_q, d] over the paged cache; returns [n, n_q * d]."""
    l = require_gpu()
    _dense(q, "q")
    n, n_q, d = q.shape
    _dense(k_pool, "k_pool", q.dtype), _dense(v_pool, "v_pool", q.dtype)
    n_pages, n_kv, page_size, pool_d = k_pool.shape
    if pool_d != d or v_pool.shape != k_pool.shape:
        raise KernelError(f"cache pools {tuple(k_pool.shape)} do not fit head_dim {d}")
    for t, name in ((tok_pos, "tok_pos"), (tok_slot, "tok_slot"), (block_table, "block_table"), (status, "status")):
        _dense(t, name, torch.int32)
    out = torch.empty((n, n_q * d), dtype=q.dtype, device=q.device)
    check(l.gi_attention_generic(_ptr(q), _ptr(k_pool), _ptr(v_pool), code(q.dtype), _ptr(block_table),
                                 _ptr(tok_pos), _ptr(tok_slot), _ptr(out), n, n_q, n_kv, d, page_size,
                                 block_table.shape[1], n_pages, int(window or 0), float(scale), _ptr(status),
                                 _stream()), l)
    return out


def sgemm_nt(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a [M,K] . w[N,K]^T in true float32."""
    l = require_gpu()
    _dense(a, "a", torch.float32), _dense(w, "w", torch.float32)
    (m, k), (n, k2) = a.shape, w.shape
    if k != k2:
        raise KernelError(f"inner sizes differ: a {tuple(a.shape)}, w {tuple(w.shape)}")
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=a.device)
    _dense(out, "out", torch.float32)
    check(l.gi_sgemm_nt(_ptr(a), _ptr(w), _ptr(out), m, n, k, k, n, _stream()), l)
    return out


def gemv_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """x [M<=8, K] . w[N,K]^T, bfloat16 operands, float32 accumulation."""
    l = require_gpu()
    _dense(x, "x", torch.bfloat16), _dense(w, "w", torch.bfloat16)
    (m, k), (n, k2) = x.shape, w.shape
    if k != k2:
        raise KernelError(f"inner sizes differ: x {tuple(x.shape)}, w {tuple(w.shape)}")
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    check(l.gi_gemv_bf16(_ptr(x), _ptr(w), _ptr(out), code(out_dtype), m, n, k, _stream()), l)
    return out


def gemm_skinny_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, n_split: int = 0,
                     wide: int = -1) -> torch.Tensor:
    """x [M<=16, K] . w[N,K]^T on the tensor cores with W streamed once.  K is shared by a cluster of
    `n_split` CTAs (1 to 8; 0: chosen from the sizes); `wide` picks 64 (1) or 32 (0) rows of W per
    CTA (-1: chosen from the sizes)."""
    l = require_gpu()
    _dense(x, "x", torch.bfloat16), _dense(w, "w", torch.bfloat16)
    (m, k), (n, k2) = x.shape, w.shape
    if k != k2:
        raise KernelError(f"inner sizes differ: x {tuple(x.shape)}, w {tuple(w.shape)}")
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    check(l.gi_gemm_skinny_bf16(_ptr(x), _ptr(w), _ptr(out), code(out_dtype), m, n, k, n_split, wide, _stream()), l)
    return out


def gemv_swiglu_bf16(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x . Wg^T) * (x . Wu^T) for one row x [1, K]: the bandwidth kernel with a gate and an up row per warp
    and the activation at its end.  Returns [1, I] bfloat16, the bits of `swiglu(gemv_bf16(x, w_gate_up))`."""
    l = require_gpu()
    _dense(x, "x", torch.bfloat16), _dense(w_gate_up, "w_gate_up", torch.bfloat16)
    (m, k), (n2, k2) = x.shape, w_gate_up.shape
    if m != 1 or k != k2:
        raise KernelError(f"gemv_swiglu_bf16 takes one row: x {tuple(x.shape)}, w {tuple(w_gate_up.shape)}")
    out = torch.empty((1, n2 // 2), dtype=torch.bfloat16, device=x.device)
    check(l.gi_gemv_swiglu_bf16(_ptr(x), _ptr(w_gate_up), _ptr(out), n2, k, _stream()), l)
    return out


def gemm_skinny_swiglu_bf16(x: torch.Tensor, w_gate_up: torch.Tensor, n_split: int = 0, wide: int = -1) -> torch.Tensor:
    """silu(x . Wg^T) * (x . Wu^T) for x [M<=16, K] and w_gate_up = [Wg; Wu] ([2 I, K], the gate first) with the
    activation in the last step of the skinny product.  Returns [M, I] bfloat16: `swiglu(gemm_skinny_bf16(x,
    w_gate_up))` up to the rounding of the sums (the kernels walk K in different orders)."""
    l = require_gpu()
    _dense(x, "x", torch.bfloat16), _dense(w_gate_up, "w_gate_up", torch.bfloat16)
    (m, k), (n2, k2) = x.shape, w_gate_up.shape
    if k != k2:
        raise KernelError(f"inner sizes differ: x {tuple(x.shape)}, w {tuple(w_gate_up.shape)}")
    out = torch.empty((m, n2 // 2), dtype=torch.bfloat16, device=x.device)
    check(l.gi_gemm_skinny_swiglu_bf16(_ptr(x), _ptr(w_gate_up), _ptr(out), m, n2, k, n_split, wide, _stream()), l)
    return out


_tcgen05_flag: dict = {}


def tcgen05_error_flag(device) -> torch.Tensor:
    """The int32 on `device` that the tcgen05 product sets when one of its bounded waits runs out."""
    key = torch.device(device).index or 0
    if key not in _tcgen05_flag:
        _tcgen05_flag[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tcgen05_flag[key]


class WaitRanOut(RuntimeError):
    """A kernel gave up one of its bounded waits; what it was writing is unspecified."""


def check_bounded_waits(device) -> None:
    """Raise `WaitRanOut` if a tcgen05 kernel launched on `device` since the last check gave up a bounded wait
    (synchronises).  The flag is cleared and the stream-K product's hand-over flags are zeroed, since a kernel
    that gave up may have left some of them set: the next call starts clean."""
    flag = tcgen05_error_flag(device)
    code = int(flag.item())
    if code:
        flag.zero_()
        key = torch.device(device).index or 0
        if key in _streamk_space:
            _streamk_space[key][1].zero_()
        raise WaitRanOut(f"a tcgen05 kernel gave up a bounded wait (code {code}: 11-13 product, 21-23 attention, "
                         "24 unmapped page, 31-33 stream-K product, 34 a partial sum that was never announced)")


def streamk_test_unanswered_flags(limit: int) -> None:
    """For the test of the bounded wait: with `limit` > 0 the stream-K product's hand-over flags are held back
    and the wait for them gives up after `limit` polls (see the kernel file); 0 restores the product."""
    require_gpu().gi_gemm_streamk_test_unanswered_flags(int(limit))


def gemm_tcgen05_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """x [M, K] . w[N, K]^T for many rows on tcgen05 tensor cores (TMA-fed, accumulators in tensor memory)."""
    l = require_gpu()
    _dense(x, "x", torch.bfloat16), _dense(w, "w", torch.bfloat16)
    (m, k), (n, k2) = x.shape, w.shape
    if k != k2:
        raise KernelError(f"inner sizes differ: x {tuple(x.shape)}, w {tuple(w.shape)}")
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    check(l.gi_gemm_tcgen05_bf16(_ptr(x), _ptr(w), _ptr(out), code(out_dtype), m, n, k,
                                 _ptr(tcgen05_error_flag(x.device)), _stream()), l)
    return out


_streamk_space: dict = {}


def _streamk_workspace(device):
    """Per device: the float32 slots through which the CTAs of the stream-K product hand over partial tiles,
    and their flags (zero between calls: every call clears what it set)."""
    key = torch.device(device).index or 0
    if key not in _streamk_space:
        l = require_gpu()
        _streamk_space[key] = (torch.empty(l.gi_gemm_streamk_workspace_floats(), dtype=torch.float32, device=device),
                               torch.zeros(l.gi_gemm_streamk_flags(), dtype=torch.int32, device=device))
    return _streamk_space[key]


def gemm_streamk_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """x [M<=64, K] . w[N,K]^T on tcgen05 with W cut evenly over the SMs (TMA-fed, operands swapped: the rows of
    W fill the 128-row side of the instruction).  Calls on one device share a work space, so they must not
    overlap (they do not on one stream)."""
    l = require_gpu()
    _dense(x, "x", torch.bfloat16), _dense(w, "w", torch.bfloat16)
    (m, k), (n, k2) = x.shape, w.shape
    if k != k2:
        raise KernelError(f"inner sizes differ: x {tuple(x.shape)}, w {tuple(w.shape)}")
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    partials, flags = _streamk_workspace(x.device)
    check(l.gi_gemm_streamk_bf16(_ptr(x), _ptr(w), _ptr(out), code(out_dtype), m, n, k, _ptr(partials), _ptr(flags),
                                 _ptr(tcgen05_error_flag(x.device)), _stream()), l)
    return out


def gemm_tcgen05_swiglu_bf16(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x . Wg^T) * (x . Wu^T) for w_gate_up = [Wg; Wu] ([2 I, K], the gate first): the gate/up product of
    a SwiGLU feed-forward with the activation in the epilogue of the tcgen05 product (pairs of CTAs).
    Returns [M, I] bfloat16, the bits of `swiglu(gemm_tcgen05_bf16(x, w_gate_up))`."""
    l = require_gpu()
    _dense(x, "x", torch.bfloat16), _dense(w_gate_up, "w_gate_up", torch.bfloat16)
    (m, k), (n2, k2) = x.shape, w_gate_up.shape
    if k != k2:
        raise KernelError(f"inner sizes differ: x {tuple(x.shape)}, w {tuple(w_gate_up.shape)}")
    out = torch.empty((m, n2 // 2), dtype=torch.bfloat16, device=x.device)
    check(l.gi_gemm_tcgen05_swiglu_bf16(_ptr(x), _ptr(w_gate_up), _ptr(out), m, n2, k,
                                        _ptr(tcgen05_error_flag(x.device)), _stream()), l)
    return out


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], streams: Optional[torch.Tensor],
           counters: Optional[torch.Tensor], seed: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 logits [n, vocab]: greedy where temperature <= 0 (or None),
    else a draw from softmax(logits / temperature) keyed by (seed, streams[row], counters[row])."""
    l = require_gpu()
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("logits must be [rows, vocab] with dense rows")
    if not logits.is_cuda or logits.dtype != torch.float32:
        raise KernelError("logits must be float32 on the GPU")
    n, vocab = logits.shape
    if temperature is not None:
        _dense(temperature, "temperature", torch.float32)
    if streams is not None:
        _dense(streams, "streams", torch.int64)
    if counters is not None:
        _dense(counters, "counters", torch.int32)
    for t, name in ((temperature, "temperature"), (streams, "streams"), (counters, "counters")):
        if t is not None and t.numel() < n:
            raise KernelError(f"{name} has fewer entries than logits has rows")
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _dense(out, "out", torch.int32)
    n_chunks = l.gi_sample_chunks(vocab)
    part_v = torch.empty((n * n_chunks,), dtype=torch.float32, device=logits.device)
    part_i = torch.empty((n * n_chunks,), dtype=torch.int32, device=logits.device)
    check(l.gi_sample(_ptr(logits), logits.stride(0), n, vocab, _ptr(temperature), _ptr(streams), _ptr(counters),
                      int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(part_v), _ptr(part_i), _ptr(out), _stream()), l)
    counters_mod.launches += 1                               # the second pass
    return out


def mma_attention_takes(dtype: torch.dtype, head_dim: int) -> bool:
    """Whether the tensor-core attention kernels take this element type and head size."""
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 128


def attention_prefill_bf16(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                           q_tiles: torch.Tensor, scale: float, window: int, rows_covered: bool = False) -> torch.Tensor:
    """Flash attention of q [n, n_q, d] over the paged cache for steps with several tokens per sequence.
    `q_tiles` int32 [n_tiles, 4] cuts the rows into runs of at most 64 consecutive tokens of one
    sequence: {slot, first row, rows, position of the first row}.  Returns [n, n_q * d]."""
    l = require_gpu()
    _dense(q, "q", torch.bfloat16), _dense(k_pool, "k_pool", torch.bfloat16), _dense(v_pool, "v_pool", torch.bfloat16)
    _dense(block_table, "block_table", torch.int32), _dense(q_tiles, "q_tiles", torch.int32)
    n, n_q, d = q.shape
    n_pages, n_kv, page_size, pool_d = k_pool.shape
    if pool_d != d or v_pool.shape != k_pool.shape:
        raise KernelError(f"cache pools {tuple(k_pool.shape)} do not fit head_dim {d}")
    if q_tiles.dim() != 2 or q_tiles.shape[1] != 4 or q_tiles.data_ptr() % 16:
        raise KernelError("q_tiles must be int32 [n_tiles, 4] starting on 16 bytes")
    # rows in no tile (padding) stay zero; when the caller says that every row lies in a tile, nothing is filled
    out = (torch.empty if rows_covered else torch.zeros)((n, n_q * d), dtype=q.dtype, device=q.device)
    check(l.gi_attention_prefill_bf16(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), _ptr(q_tiles),
                                      q_tiles.shape[0], _ptr(out), n_q, n_kv, d, page_size, block_table.shape[1],
                                      n_pages, int(window or 0), float(scale), _stream()), l)
    return out


def tcgen05_attention_takes(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill attention takes this element type, head size and page size."""
    return dtype == torch.bfloat16 and head_dim == 128 and page_size % 64 == 0


def attention_prefill_tcgen05(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                              q_tiles128: torch.Tensor, scale: float, window: int, rows_covered: bool = False) -> torch.Tensor:
    """Flash attention of q [n, n_q, 128] over the paged cache on tcgen05 tensor cores (TMA-fed, S, P and
    P V in tensor memory).  `q_tiles128` int32 [n_tiles, 4] cuts the rows into runs of at most 128
    consecutive tokens of one sequence: {slot, first row, rows, position of the first row}."""
    l = require_gpu()
    _dense(q, "q", torch.bfloat16), _dense(k_pool, "k_pool", torch.bfloat16), _dense(v_pool, "v_pool", torch.bfloat16)
    _dense(block_table, "block_table", torch.int32), _dense(q_tiles128, "q_tiles128", torch.int32)
    n, n_q, d = q.shape
    n_pages, n_kv, page_size, pool_d = k_pool.shape
    if pool_d != d or v_pool.shape != k_pool.shape:
        raise KernelError(f"cache pools {tuple(k_pool.shape)} do not fit head_dim {d}")
    if q_tiles128.dim() != 2 or q_tiles128.shape[1] != 4 or q_tiles128.data_ptr() % 16:
        raise KernelError("q_tiles128 must be int32 [n_tiles, 4] starting on 16 bytes")
    # rows in no tile (padding) stay zero; when the caller says that every row lies in a tile, nothing is filled
    out = (torch.empty if rows_covered else torch.zeros)((n, n_q * d), dtype=q.dtype, device=q.device)
    check(l.gi_attention_prefill_tcgen05(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), _ptr(q_tiles128),
                                         q_tiles128.shape[0], _ptr(out), n, n_q, n_kv, d, page_size,
                                         block_table.shape[1], n_pages, int(window or 0), float(scale),
                                         _ptr(tcgen05_error_flag(q.device)), _stream()), l)
    return out


def decode_splits(n_seqs: int, n_kv: int) -> int:
    """Slices of the keys per (sequence, key/value head) in the decode kernel.  Measured on a B200 at
    2,048 and 4,096 cached tokens (8 key/value heads): about 256 CTAs are wanted at small batches (but at
    most 16 slices); three slices are best between 64 and 512 (sequence, head) pairs (batches 16 and 32:
    5 to 12 % better than two), and two slices still pay when the batch alone makes several hundred CTAs,
    because they even out the last wave.  The count is fixed per batch size: a recorded step is replayed
    while the sequences grow."""
    pairs = max(1, n_seqs * n_kv)
    if pairs <= 64:
        return max(1, min(16, -(-256 // pairs)))
    if pairs < 512:
        return 3
    return 2 if pairs < 1776 else 1


def decode_splits_tcgen05(n_seqs: int, n_kv: int) -> int:
    """Slices of the keys per (sequence, key/value head) in the tcgen05 decode kernel.  Measured on a B200 at
    2,048 and 4,096 cached tokens (8 key/value heads): about 256 CTAs at small batches (16 slices at batch 1,
    4 at batch 8, 2 at batch 16) and no slicing from 256 (sequence, head) pairs on (batch 64: 86 us whole
    against 93 us in two slices).  Fixed per batch size: a recorded step is replayed while the sequences grow."""
    return max(1, min(16, -(-256 // max(1, n_seqs * n_kv))))


def tcgen05_decode_takes(dtype: torch.dtype, head_dim: int, page_size: int, group: int) -> bool:
    return dtype == torch.bfloat16 and head_dim == 128 and page_size % 64 == 0 and group <= 16


def attention_decode_tcgen05(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                             tok_pos: torch.Tensor, tok_slot: torch.Tensor, scale: float, window: int,
                             n_splits: Optional[int] = None) -> torch.Tensor:
    """Split-KV attention for decode steps on TMA and tcgen05: the arguments of `attention_decode_bf16`; heads
    of 128, pages that are a multiple of 64 tokens, at most 16 query heads per key/value head."""
    l = require_gpu()
    _dense(q, "q", torch.bfloat16), _dense(k_pool, "k_pool", torch.bfloat16), _dense(v_pool, "v_pool", torch.bfloat16)
    for t, name in ((tok_pos, "tok_pos"), (tok_slot, "tok_slot"), (block_table, "block_table")):
        _dense(t, name, torch.int32)
    n, n_q, d = q.shape
    n_pages, n_kv, page_size, pool_d = k_pool.shape
    if pool_d != d or v_pool.shape != k_pool.shape:
        raise KernelError(f"cache pools {tuple(k_pool.shape)} do not fit head_dim {d}")
    if tok_pos.numel() < n or tok_slot.numel() < n:
        raise KernelError("tok_pos / tok_slot are shorter than the token rows")
    n_splits = n_splits or decode_splits_tcgen05(n, n_kv)
    out = torch.empty((n, n_q * d), dtype=q.dtype, device=q.device)
    part_o = part_ml = None
    if n_splits > 1:
        part_o = torch.empty((n * n_q * n_splits * d,), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n * n_q * n_splits * 2,), dtype=torch.float32, device=q.device)
    check(l.gi_attention_decode_tcgen05(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), _ptr(tok_pos),
                                        _ptr(tok_slot), _ptr(part_o), _ptr(part_ml), _ptr(out), n, n_q, n_kv, d, page_size,
                                        block_table.shape[1], n_pages, int(window or 0), float(scale), n_splits,
                                        _ptr(tcgen05_error_flag(q.device)), _stream()), l)
    if n_splits > 1:                                 # one slice: the kernel wrote the output itself
        check(l.gi_attention_decode_combine(_ptr(part_o), _ptr(part_ml), _ptr(out), n * n_q, d, n_splits, _stream()), l)
    return out


def attention_decode_bf16(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                          tok_pos: torch.Tensor, tok_slot: torch.Tensor, scale: float, window: int,
                          n_splits: Optional[int] = None) -> torch.Tensor:
    """Split-KV attention for decode steps: q [n_seqs, n_q, d], one token per sequence at position
    tok_pos (the key at that position is already in the cache).  Returns [n_seqs, n_q * d].
    The partial results of the slices go through scratch memory allocated here."""
    l = require_gpu()
    _dense(q, "q", torch.bfloat16), _dense(k_pool, "k_pool", torch.bfloat16), _dense(v_pool, "v_pool", torch.bfloat16)
    for t, name in ((tok_pos, "tok_pos"), (tok_slot, "tok_slot"), (block_table, "block_table")):
        _dense(t, name, torch.int32)
    n, n_q, d = q.shape
    n_pages, n_kv, page_size, pool_d = k_pool.shape
    if pool_d != d or v_pool.shape != k_pool.shape:
        raise KernelError(f"cache pools {tuple(k_pool.shape)} do not fit head_dim {d}")
    if tok_pos.numel() < n or tok_slot.numel() < n:
        raise KernelError("tok_pos / tok_slot are shorter than the token rows")
    n_splits = n_splits or decode_splits(n, n_kv)
    out = torch.empty((n, n_q * d), dtype=q.dtype, device=q.device)
    part_o = torch.empty((n * n_q * n_splits * d,), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((n * n_q * n_splits * 2,), dtype=torch.float32, device=q.device)
    check(l.gi_attention_decode_bf16(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), _ptr(tok_pos),
                                     _ptr(tok_slot), _ptr(out), _ptr(part_o), _ptr(part_ml), n, n_q, n_kv, d,
                                     page_size, block_table.shape[1], n_pages, int(window or 0), float(scale),
                                     n_splits, _stream()), l)
    counters.launches += 1                                   # the combine kernel
    return out
