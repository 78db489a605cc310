"""Where the time of a recorded decode step goes, kernel by kernel, with the overlap between kernels in it.

    python -m garlic_inference_b200.engine.timeline [--batch 8] [--cached 2048] [--layers N] [--config config.json]

Builds the library a second time with its timeline hooks (csrc/common.cuh; the ordinary build has none and is
not touched), decodes with random weights and prints, for one replayed step, every kernel's launch size, when
its first block started, when the kernel before it had finished ("released"), and how long it took from there
until the next kernel was released: the last column adds up to the step.  Kernels that were launched while
their predecessor still ran show it in the lead (released - start), the time their blocks had for fetching
what does not depend on the predecessor.  A summary gives the medians per position in the repeating layer
(for the default architecture: norm, q/k/v product, rotary + append, attention, combine, o product, norm,
gate/up product with SwiGLU, down product).  Without --config the sizes are the benchmark's (bench.py).
"""
from __future__ import annotations

import argparse
import ctypes
import os
import statistics
import sys

import torch

ENTRIES = 4096


def attach(device) -> torch.Tensor:
    """Give every file of the library the buffer its kernels write their marks to."""
    from ..csrc import build
    from ..ops import require_gpu
    lib = require_gpu()
    buf = torch.zeros(4 + 4 * ENTRIES, dtype=torch.int64, device=device)
    for src in build.sources():
        fn = getattr(lib, "gi_tl_set_" + src.stem)
        fn.argtypes, fn.restype = [ctypes.c_void_p], None
        fn(buf.data_ptr())
    return buf


def read(buf: torch.Tensor) -> list[tuple[int, int, float, float]]:
    """(blocks, threads, start us, released us) per kernel, in launch order, from the first kernel's start."""
    b = buf.cpu().tolist()
    n = min(b[0], b[1], ENTRIES)
    if n == 0:
        return []
    t0 = b[4]
    return [(b[4 + 4 * i + 2] >> 16, b[4 + 4 * i + 2] & 0xFFFF, (b[4 + 4 * i] - t0) / 1e3, (b[4 + 4 * i + 1] - t0) / 1e3)
            for i in range(n)]


def period(tags: list) -> int:
    """The length of the repeating run of launch sizes in the middle of the step (a layer), 0 if none."""
    n = len(tags)
    lo, hi = n // 4, 3 * n // 4
    for p in range(2, max(2, n // 3)):
        if all(tags[i] == tags[i + p] for i in range(lo, hi - p)):
            return p
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--cached", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--config", default=None, help="a config.json; default: the benchmark's sizes")
    ap.add_argument("--all", action="store_true", help="print every kernel, not only the summary and two layers")
    args = ap.parse_args(argv)
    os.environ["GARLIC_B200_TIMELINE"] = "1"      # before anything builds or loads the library: the build with hooks

    import json
    from .. import LanguageModel
    from ..config.registry import config_class_for
    from ..sampling import SamplingParams
    if args.config:
        with open(args.config) as f:
            raw = json.load(f)
    else:
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
        import bench
        raw = dict(bench.QWEN3_8B, architectures=["Qwen3ForCausalLM"])
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = config_class_for(raw["architectures"][0]).from_dict(raw)
    per_seq = -(-(args.cached + 64) // 64) * 64
    model = LanguageModel.from_random(cfg, seed=0, device=0, dtype="bfloat16", max_tokens=args.batch * per_seq + 64)
    buf = attach(model.model.rt.device)
    eng, sampler, greedy = model.engine, model.sampler, SamplingParams()
    gen = torch.Generator().manual_seed(0)
    slots, firsts = [], []
    for _ in range(args.batch):
        s = eng.alloc_slot()
        prompt = torch.randint(0, cfg.vocab_size, (args.cached,), generator=gen).tolist()
        firsts.append(sampler.sample(model.step([(s, prompt, [args.cached - 1])]), greedy, [0], [0]))
        slots.append(s)
    toks = torch.cat(firsts)
    for _ in range(40):                                   # past the slow steps that follow the prompt passes
        toks = sampler.sample(eng.step_decode_device(slots, toks), greedy, slots, slots)
    torch.cuda.synchronize()
    buf.zero_()
    torch.cuda.synchronize()
    sampler.sample(eng.step_decode_device(slots, toks), greedy, slots, slots)
    torch.cuda.synchronize()
    rows = read(buf)
    if not rows:
        print("no marks: the library was not built with its timeline hooks")
        return 1
    cost = [rows[i + 1][3] - rows[i][3] for i in range(len(rows) - 1)] + [0.0]
    tags = [(r[0], r[1]) for r in rows]
    p = period(tags)
    print(f"{len(rows)} kernels, {rows[-1][3]:.1f} us from the first start to the last release; "
          f"a layer is {p} kernels" if p else f"{len(rows)} kernels")
    header = "  idx  blocks x threads   start us  released us   lead us   until the next release us"
    show = range(len(rows)) if args.all or not p else list(range(0, min(len(rows), 1 + 2 * p))) + list(range(len(rows) - 6, len(rows)))
    print(header)
    for i in show:
        r = rows[i]
        print(f"{i:5d} {r[0]:7d} x {r[1]:4d} {r[2]:12.2f} {r[3]:12.2f} {r[3] - r[2]:9.2f} {cost[i]:12.2f}")
    if p:
        first = next(i for i in range(len(rows) - 2 * p) if all(tags[j] == tags[j + p] for j in range(i, i + p)))
        n_layers = 1
        while first + (n_layers + 1) * p <= len(rows) and all(tags[first + n_layers * p + j] == tags[first + j] for j in range(p)):
            n_layers += 1
        print(f"medians over layers 2 to {n_layers - 1} of {n_layers}, by position in the layer:")
        total = 0.0
        for j in range(p):
            c = [cost[first + l * p + j] for l in range(1, n_layers - 1)]
            lead = [rows[first + l * p + j][3] - rows[first + l * p + j][2] for l in range(1, n_layers - 1)]
            r = rows[first + p + j]
            total += statistics.median(c)
            print(f"   {j:2d} {r[0]:7d} x {r[1]:4d}  {statistics.median(c):7.2f} us   lead {statistics.median(lead):6.2f} us")
        print(f"   a layer: {total:.2f} us")
    return 0


if __name__ == "__main__":
    sys.exit(main())
