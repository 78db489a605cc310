"""Single kernels at the benchmark model's sizes, for timing and for profilers.

    python -m garlic_inference_b200.ops.microbench run  OP M [SHAPE]     a few plain launches (what ncu captures)
    python -m garlic_inference_b200.ops.microbench time [linear|attn|prefill|small]   GPU time inside CUDA graphs, cold L2
    python -m garlic_inference_b200.ops.microbench time attn_long    the attention kernels at 8,192 to 32,768 tokens

OP: gemv | skinny | streamk | cublas | tcgen05 (M = rows of x, SHAPE = qkv | o | gate_up | down | lm_head at Qwen3-8B sizes),
attn_decode and attn_decode_tcgen05 (M = sequences, 2,048 cached tokens each), attn_prefill and attn_prefill_tcgen05 (M = prompt length).
`time` rotates over several copies of the operands (more than the 126 MB of L2) and reports the
algorithmic bytes over the time.
"""
from __future__ import annotations

import sys

import torch

from . import kernels

SHAPES = {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (24576, 4096), "down": (4096, 12288),
          "lm_head": (151936, 4096)}
N_Q, N_KV, HEAD_DIM, PAGE = 32, 8, 128, 64
DEV = "cuda"


def graph_time(fns, reps: int = 5) -> float:
    """Milliseconds per call of the callables captured back to back in one CUDA graph."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for f in fns:
            f()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for f in fns:
            f()
    graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        graph.replay()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / reps / len(fns)


def _weights(shape: str, copies: int):
    n, k = SHAPES[shape]
    return [torch.randn(n, k, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]


def _linear(op: str, x, w):
    if op == "gemv":
        return kernels.gemv_bf16(x, w, torch.bfloat16)
    if op == "skinny":
        return kernels.gemm_skinny_bf16(x, w, torch.bfloat16)
    if op == "cublas":
        return torch.mm(x, w.t())
    if op == "tcgen05":
        return kernels.gemm_tcgen05_bf16(x, w, torch.bfloat16)
    if op == "streamk":
        return kernels.gemm_streamk_bf16(x, w, torch.bfloat16)
    raise SystemExit(f"unknown op {op}")


def _decode_case(batch: int, ctx: int, copies: int):
    n_pages = batch * ctx // PAGE
    pools = [(torch.randn(n_pages, N_KV, PAGE, HEAD_DIM, device=DEV, dtype=torch.bfloat16),
              torch.randn(n_pages, N_KV, PAGE, HEAD_DIM, device=DEV, dtype=torch.bfloat16)) for _ in range(copies)]
    table = torch.arange(n_pages, dtype=torch.int32, device=DEV).view(batch, -1)
    q = torch.randn(batch, N_Q, HEAD_DIM, device=DEV, dtype=torch.bfloat16)
    pos = torch.full((batch,), ctx - 1, dtype=torch.int32, device=DEV)
    slot = torch.arange(batch, dtype=torch.int32, device=DEV)
    return pools, table, q, pos, slot


def run(op: str, m: int, shape: str = "gate_up") -> None:
    if op in ("gemv", "skinny", "cublas", "tcgen05", "streamk"):
        ws = _weights(shape, 3)
        x = torch.randn(m, SHAPES[shape][1], device=DEV, dtype=torch.bfloat16)
        for i in range(6):
            _linear(op, x, ws[i % 3])
    elif op == "attn_decode":
        pools, table, q, pos, slot = _decode_case(m, 2048, 2)
        for i in range(6):
            kernels.attention_decode_bf16(q, pools[i % 2][0], pools[i % 2][1], table, pos, slot, HEAD_DIM ** -0.5, 0)
    elif op == "attn_decode_tcgen05":
        pools, table, q, pos, slot = _decode_case(m, 2048, 2)
        for i in range(6):
            kernels.attention_decode_tcgen05(q, pools[i % 2][0], pools[i % 2][1], table, pos, slot, HEAD_DIM ** -0.5, 0)
        print("error flag", int(kernels.tcgen05_error_flag(DEV).item()))
    elif op == "attn_prefill":
        n_pages = -(-m // PAGE)
        k_pool = torch.randn(n_pages, N_KV, PAGE, HEAD_DIM, device=DEV, dtype=torch.bfloat16)
        v_pool = torch.randn_like(k_pool)
        table = torch.arange(n_pages, dtype=torch.int32, device=DEV).view(1, -1)
        q = torch.randn(m, N_Q, HEAD_DIM, device=DEV, dtype=torch.bfloat16)
        tiles = torch.tensor([(0, r, min(64, m - r), r) for r in range(0, m, 64)], dtype=torch.int32, device=DEV)
        for _ in range(4):
            kernels.attention_prefill_bf16(q, k_pool, v_pool, table, tiles, HEAD_DIM ** -0.5, 0)
    elif op == "attn_prefill_tcgen05":
        n_pages = -(-m // PAGE)
        k_pool = torch.randn(n_pages, N_KV, PAGE, HEAD_DIM, device=DEV, dtype=torch.bfloat16)
        v_pool = torch.randn_like(k_pool)
        table = torch.arange(n_pages, dtype=torch.int32, device=DEV).view(1, -1)
        q = torch.randn(m, N_Q, HEAD_DIM, device=DEV, dtype=torch.bfloat16)
        tiles = torch.tensor([(0, r, min(128, m - r), r) for r in reversed(range(0, m, 128))], dtype=torch.int32, device=DEV)
        for _ in range(4):
            kernels.attention_prefill_tcgen05(q, k_pool, v_pool, table, tiles, HEAD_DIM ** -0.5, 0)
        print("error flag", int(kernels.tcgen05_error_flag(DEV).item()))
    else:
        raise SystemExit(f"unknown op {op}")
    torch.cuda.synchronize()
    print("ok")


def time_linear() -> None:
    for shape, (n, k) in SHAPES.items():
        copies = 2 if shape == "lm_head" else max(3, int(500e6 // (n * k * 2)) + 1)
        ws = _weights(shape, copies)
        for m in (1, 2, 4, 8, 16, 32, 64):
            x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
            ops = (["gemv"] if m <= 8 else []) + (["skinny"] if m <= 16 else []) + ["streamk", "cublas"]
            res = {op: graph_time([(lambda w=w, op=op: _linear(op, x, w)) for w in ws]) for op in ops}
            print(f"{shape:8s} M={m:3d}  " + "  ".join(f"{op}: {ms * 1e3:7.1f} us {n * k * 2 / ms / 1e6:5.0f} GB/s"
                                                        for op, ms in res.items()), flush=True)
        del ws


def time_attention() -> None:
    for batch in (1, 8, 64):
        for ctx in (2048, 4096):
            nbytes = batch * ctx * N_KV * HEAD_DIM * 2 * 2
            copies = min(40, max(3, int(500e6 // nbytes) + 1))
            pools, table, q, pos, slot = _decode_case(batch, ctx, copies)
            ms = graph_time([(lambda p=p: kernels.attention_decode_bf16(q, p[0], p[1], table, pos, slot,
                                                                         HEAD_DIM ** -0.5, 0)) for p in pools])
            ms2 = graph_time([(lambda p=p: kernels.attention_decode_tcgen05(q, p[0], p[1], table, pos, slot,
                                                                            HEAD_DIM ** -0.5, 0)) for p in pools])
            print(f"attn_decode batch={batch:3d} ctx={ctx}  mma.sync {ms * 1e3:7.1f} us  {nbytes / ms / 1e6:5.0f} GB/s  "
                  f"tcgen05 {ms2 * 1e3:7.1f} us  {nbytes / ms2 / 1e6:5.0f} GB/s  "
                  f"(slices {kernels.decode_splits(batch, N_KV)} / {kernels.decode_splits_tcgen05(batch, N_KV)})", flush=True)
            del pools


def time_attention_long() -> None:
    """The tcgen05 attention kernels beyond the benchmark's lengths: decode over 8,192 to 32,768 cached tokens at
    small batches (the slices are the ones the engine picks for the batch), one prompt of 8,192 and of 16,384 tokens."""
    for batch in (1, 2, 4, 8):
        for ctx in (8192, 16384, 32768):
            nbytes = batch * ctx * N_KV * HEAD_DIM * 2 * 2
            copies = min(40, max(3, int(500e6 // nbytes) + 1))
            pools, table, q, pos, slot = _decode_case(batch, ctx, copies)
            ms = graph_time([(lambda p=p: kernels.attention_decode_tcgen05(q, p[0], p[1], table, pos, slot,
                                                                           HEAD_DIM ** -0.5, 0)) for p in pools])
            print(f"attn_decode batch={batch:3d} ctx={ctx:6d}  tcgen05 {ms * 1e3:7.1f} us  {nbytes / ms / 1e6:5.0f} GB/s  "
                  f"({kernels.decode_splits_tcgen05(batch, N_KV)} slices)", flush=True)
            del pools
    for m in (8192, 16384):
        n_pages = m // PAGE
        k_pool = torch.randn(n_pages, N_KV, PAGE, HEAD_DIM, device=DEV, dtype=torch.bfloat16)
        v_pool = torch.randn_like(k_pool)
        table = torch.arange(n_pages, dtype=torch.int32, device=DEV).view(1, -1)
        q = torch.randn(m, N_Q, HEAD_DIM, device=DEV, dtype=torch.bfloat16)
        tiles = torch.tensor([(0, r, 128, r) for r in reversed(range(0, m, 128))], dtype=torch.int32, device=DEV)
        ms = graph_time([lambda: kernels.attention_prefill_tcgen05(q, k_pool, v_pool, table, tiles, HEAD_DIM ** -0.5, 0)] * 3)
        flops = 4 * N_Q * HEAD_DIM * m * (m + 128) / 2
        print(f"attention prompt of {m}  tcgen05 {ms * 1e3:8.1f} us  {flops / ms / 1e9:5.0f} TFLOP/s", flush=True)
    print("error flag", int(kernels.tcgen05_error_flag(DEV).item()))


def time_small(hidden: int = 4096, inter: int = 12288) -> None:
    """The kernels between the products of a decode step, 32 calls back to back in a graph on operands
    that stay in L2 (as they do in a step, where the kernel before has just written them)."""
    for m in (1, 8, 64):
        res = torch.randn(m, hidden, device=DEV)
        delta = torch.randn(m, hidden, device=DEV, dtype=torch.bfloat16)
        w = torch.ones(hidden, device=DEV, dtype=torch.bfloat16)
        gate_up = torch.randn(m, 2 * inter, device=DEV, dtype=torch.bfloat16)
        qkv = torch.randn(m, (N_Q + 2 * N_KV) * HEAD_DIM, device=DEV, dtype=torch.bfloat16)
        wn = torch.ones(HEAD_DIM, device=DEV, dtype=torch.bfloat16)
        ctx = 2048
        pools, table, _, pos, slot = _decode_case(m, ctx, 1)
        cos = torch.randn(ctx, HEAD_DIM // 2, device=DEV)
        sin = torch.randn(ctx, HEAD_DIM // 2, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        times = {
            "add_rmsnorm": graph_time([lambda: kernels.add_rmsnorm(delta, res, w, 1e-6, torch.bfloat16)] * 32),
            "swiglu": graph_time([lambda: kernels.swiglu(gate_up)] * 32),
            "qk_norm_rope_append": graph_time([lambda: kernels.qk_norm_rope_append(
                qkv, N_Q, N_KV, HEAD_DIM, wn, wn, 1e-6, cos, sin, HEAD_DIM, pos, slot, pools[0][0], pools[0][1], table,
                status)] * 32),
        }
        print(f"M={m:3d}  " + "  ".join(f"{k}: {v * 1e3:5.2f} us" for k, v in times.items()), flush=True)
    # the same kernels over a prompt of 2,048 tokens (one sequence, positions 0..2047)
    m, ctx = 2048, 2048
    res = torch.randn(m, hidden, device=DEV)
    delta = torch.randn(m, hidden, device=DEV, dtype=torch.bfloat16)
    w = torch.ones(hidden, device=DEV, dtype=torch.bfloat16)
    gate_up = torch.randn(m, 2 * inter, device=DEV, dtype=torch.bfloat16)
    qkv = torch.randn(m, (N_Q + 2 * N_KV) * HEAD_DIM, device=DEV, dtype=torch.bfloat16)
    wn = torch.ones(HEAD_DIM, device=DEV, dtype=torch.bfloat16)
    pools, table, _, _, _ = _decode_case(1, ctx, 1)
    pos = torch.arange(m, dtype=torch.int32, device=DEV)
    slot = torch.zeros(m, dtype=torch.int32, device=DEV)
    cos = torch.randn(ctx, HEAD_DIM // 2, device=DEV)
    sin = torch.randn(ctx, HEAD_DIM // 2, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    times = {
        "add_rmsnorm": graph_time([lambda: kernels.add_rmsnorm(delta, res, w, 1e-6, torch.bfloat16)] * 8),
        "swiglu": graph_time([lambda: kernels.swiglu(gate_up)] * 8),
        "qk_norm_rope_append": graph_time([lambda: kernels.qk_norm_rope_append(
            qkv, N_Q, N_KV, HEAD_DIM, wn, wn, 1e-6, cos, sin, HEAD_DIM, pos, slot, pools[0][0], pools[0][1], table,
            status)] * 8),
    }
    print(f"M={m}  " + "  ".join(f"{k}: {v * 1e3:5.2f} us" for k, v in times.items()), flush=True)


def time_prefill_linear(m: int = 2048) -> None:
    """The products of a prompt of `m` tokens: this library's tcgen05 kernel against the library product."""
    for shape, (n, k) in SHAPES.items():
        if shape == "lm_head":
            continue
        ws = _weights(shape, 3)
        xs = [torch.randn(m, k, device=DEV, dtype=torch.bfloat16) for _ in range(3)]
        flops = 2.0 * m * n * k
        res = {"tcgen05": graph_time([(lambda w=w, x=x: kernels.gemm_tcgen05_bf16(x, w, torch.bfloat16)) for w, x in zip(ws, xs)]),
               "cublas": graph_time([(lambda w=w, x=x: torch.mm(x, w.t())) for w, x in zip(ws, xs)])}
        print(f"{shape:8s} M={m}  " + "  ".join(f"{op}: {ms * 1e3:7.1f} us {flops / ms / 1e9:6.0f} TFLOP/s"
                                                for op, ms in res.items()), flush=True)
    # the gate/up product with the SwiGLU in its epilogue against the library product and the SwiGLU kernel
    ws = _weights("gate_up", 3)
    xs = [torch.randn(m, SHAPES["gate_up"][1], device=DEV, dtype=torch.bfloat16) for _ in range(3)]
    res = {"tcgen05 fused": graph_time([(lambda w=w, x=x: kernels.gemm_tcgen05_swiglu_bf16(x, w)) for w, x in zip(ws, xs)]),
           "cublas + swiglu": graph_time([(lambda w=w, x=x: kernels.swiglu(torch.mm(x, w.t()))) for w, x in zip(ws, xs)])}
    print(f"gate_up+swiglu M={m}  " + "  ".join(f"{op}: {ms * 1e3:7.1f} us" for op, ms in res.items()), flush=True)
    del ws, xs
    # causal attention of the same prompt: 4 * n_q * d * m^2 / 2 flops
    n_pages = -(-m // PAGE)
    k_pool = torch.randn(n_pages, N_KV, PAGE, HEAD_DIM, device=DEV, dtype=torch.bfloat16)
    v_pool = torch.randn_like(k_pool)
    table = torch.arange(n_pages, dtype=torch.int32, device=DEV).view(1, -1)
    q = torch.randn(m, N_Q, HEAD_DIM, device=DEV, dtype=torch.bfloat16)
    # the runs with the most keys first, as the engine orders them
    t64 = torch.tensor([(0, r, min(64, m - r), r) for r in reversed(range(0, m, 64))], dtype=torch.int32, device=DEV)
    t128 = torch.tensor([(0, r, min(128, m - r), r) for r in reversed(range(0, m, 128))], dtype=torch.int32, device=DEV)
    flops = 4.0 * N_Q * HEAD_DIM * m * (m + 1) / 2
    res = {"tcgen05": graph_time([lambda: kernels.attention_prefill_tcgen05(q, k_pool, v_pool, table, t128, HEAD_DIM ** -0.5, 0)] * 3),
           "mma.sync": graph_time([lambda: kernels.attention_prefill_bf16(q, k_pool, v_pool, table, t64, HEAD_DIM ** -0.5, 0)] * 3)}
    print(f"attention M={m}  " + "  ".join(f"{op}: {ms * 1e3:7.1f} us {flops / ms / 1e9:6.0f} TFLOP/s" for op, ms in res.items()),
          flush=True)
    print("error flag", int(kernels.tcgen05_error_flag(DEV).item()))


def main(argv) -> int:
    if len(argv) >= 3 and argv[0] == "run":
        run(argv[1], int(argv[2]), argv[3] if len(argv) > 3 else "gate_up")
    elif argv and argv[0] == "time":
        which = argv[1] if len(argv) > 1 else "all"
        if which in ("all", "linear"):
            time_linear()
        if which in ("all", "attn"):
            time_attention()
        if which in ("all", "prefill"):
            time_prefill_linear()
        if which in ("all", "small"):
            time_small()
        if which == "attn_long":
            time_attention_long()
    else:
        print(__doc__)
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
