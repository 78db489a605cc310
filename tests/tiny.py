"""Tiny configurations, traces and comparison helpers shared by the tests.

Configurations of the architecture that differ in every size and option:
layers, width (one no power of two), heads and groups (2, 6 and 1 query heads
per key/value head), head sizes 16 / 32 / 48, feed-forward width, vocabulary,
rope theta, the norms' eps, positions, tied or separate head, and the window
(none; none; 40 keys on the two middle layers of four; none; 100 keys on the outer layers of three).
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

REPO = Path(__file__).resolve().parent.parent

TINY = {
    "A": dict(cfg=dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                       head_dim=16, intermediate_size=192, vocab_size=512, rope_theta=1e4, rms_norm_eps=1e-6,
                       max_position_embeddings=128, tie_word_embeddings=True),
              seed=0, std=0.02, norm_std=0.1),
    "B": dict(cfg=dict(hidden_size=96, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=1,
                       head_dim=32, intermediate_size=256, vocab_size=1000, rope_theta=1e6, rms_norm_eps=1e-5,
                       max_position_embeddings=256, tie_word_embeddings=False),
              seed=1, std=0.05, norm_std=0.2),
    # B with room for 640 positions (the same weights: no tensor depends on the limit), for long decoding
    "F": dict(cfg=dict(hidden_size=96, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=1,
                       head_dim=32, intermediate_size=256, vocab_size=1000, rope_theta=1e6, rms_norm_eps=1e-5,
                       max_position_embeddings=640, tie_word_embeddings=False),
              seed=1, std=0.05, norm_std=0.2),
    "C": dict(cfg=dict(hidden_size=80, num_hidden_layers=4, num_attention_heads=5, num_key_value_heads=5,
                       head_dim=48, intermediate_size=112, vocab_size=777, rope_theta=5e5, rms_norm_eps=3e-5,
                       max_position_embeddings=512, tie_word_embeddings=False, sliding_window=40,
                       layer_types=["full_attention", "sliding_attention", "sliding_attention",
                                    "full_attention"]),
              seed=2, std=0.08, norm_std=0.15),
    # heads of 128 (and, in the tests, cache pages of 64): the sizes the tcgen05 attention kernel takes
    "D": dict(cfg=dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                       head_dim=128, intermediate_size=320, vocab_size=600, rope_theta=1e6, rms_norm_eps=1e-6,
                       max_position_embeddings=1024, tie_word_embeddings=False),
              seed=3, std=0.04, norm_std=0.1),
    # heads of 128 with a window of 100 keys on the first and the last of three layers, one key/value head for
    # four query heads: the tcgen05 kernels with windows, and pages of a window group given back while decoding
    "E": dict(cfg=dict(hidden_size=192, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=1,
                       head_dim=128, intermediate_size=224, vocab_size=400, rope_theta=1e5, rms_norm_eps=2e-6,
                       max_position_embeddings=1024, tie_word_embeddings=True, sliding_window=100,
                       layer_types=["sliding_attention", "full_attention", "sliding_attention"]),
              seed=4, std=0.05, norm_std=0.1),
    # tied head, heads of 128 with four query heads per key/value head and n_heads * head_dim != hidden: what
    # upstream's own code (always tied, bfloat16) can run too; tests/golden holds its logits for A and for this
    "G": dict(cfg=dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2,
                       head_dim=128, intermediate_size=384, vocab_size=640, rope_theta=1e6, rms_norm_eps=1e-6,
                       max_position_embeddings=512, tie_word_embeddings=True),
              seed=5, std=0.04, norm_std=0.1),
}

# tolerances (never widened to pass): float32 logits against the plain float32 implementation,
# bfloat16 logits against the same, both relative to the largest logit of the comparison
TOL = {"float32": 1e-4, "bfloat16": 3e-2}


# The worst error of the engine against the plain implementation that each configuration showed when these
# numbers were recorded (all cuttings, relative to the largest logit).  A comparison may not exceed twice its
# recorded value: the flat bounds above would let a regression of ten times pass.
SEEN = {
    "bfloat16": {"A": 3.4e-3, "B": 1.14e-2, "C": 1.0e-2, "D": 9.5e-3, "E": 1.01e-2},
    # float32 showed 4e-7 to 1.3e-6 (a few steps of the last bit at the scale of the largest logit, and the plain
    # implementation's own rounding depends on the CPU it runs on): one bound of 1e-5 for all, ten times under TOL
    "float32": {"A": 5e-6, "B": 5e-6, "C": 5e-6, "D": 5e-6, "E": 5e-6},
}


def check_seen(name: str, dtype: str, worst: float) -> None:
    seen = SEEN[dtype].get(name)
    if seen is not None:
        assert worst <= 2 * seen, (f"{name} {dtype}: worst relative error {worst:.3e} is more than twice the "
                                   f"{seen:.3e} recorded for this configuration")


def make_config(name: str):
    from garlic_inference_b200 import Qwen3Config
    return Qwen3Config(**TINY[name]["cfg"])


def write_model(name: str, folder) -> Path:
    from garlic_inference_b200 import write_random_model
    t = TINY[name]
    return write_random_model(folder, make_config(name), seed=t["seed"], std=t["std"], norm_std=t["norm_std"])


def random_requests(vocab: int, lengths, seed: int) -> dict[str, list[int]]:
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, vocab, size=n).tolist() for i, n in enumerate(lengths)}


def plain_logits(model_dir, requests: dict[str, list[int]], dtype=torch.float32) -> dict[str, np.ndarray]:
    """Logits at every position of every request from the plain implementation."""
    import plain_qwen3 as plain
    cfg, weights = plain.read_model_dir(model_dir)
    return {rid: plain.forward(cfg, weights, toks, dtype).to(torch.float32).numpy()
            for rid, toks in requests.items()}


# ---- traces: lists of step records in the format of bin/trace_run ---------------------------
def trace_whole(requests, want_all=True):
    """Each request alone, its whole token list in one step."""
    steps = []
    for rid, toks in requests.items():
        want = list(range(len(toks))) if want_all else [len(toks) - 1]
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks, "want": want}], "end": [rid]})
    return steps


def trace_tail_by_one(requests, tail=32):
    """Each request alone: all but the last `tail` tokens in one step, the rest one token a step."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps),
                      "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        for i in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def trace_batched(requests, batches, prompt_frac=0.5):
    """Batches of requests that start together: a prompt part of each (unequal lengths) in one step,
    then one token each per step; shorter requests end earlier.  `batches` lists request ids."""
    steps = []
    for batch in batches:
        cut = {rid: max(1, int(len(requests[rid]) * prompt_frac)) for rid in batch}
        steps.append({"step": len(steps),
                      "entries": [{"id": rid, "tokens": requests[rid][:cut[rid]], "want": list(range(cut[rid]))}
                                  for rid in batch],
                      "end": [rid for rid in batch if cut[rid] == len(requests[rid])]})
        live = [rid for rid in batch if cut[rid] < len(requests[rid])]
        k = 0
        while live:
            entries = [{"id": rid, "tokens": [requests[rid][cut[rid] + k]], "want": [0]} for rid in live]
            ending = [rid for rid in live if cut[rid] + k == len(requests[rid]) - 1]
            steps.append({"step": len(steps), "entries": entries, "end": ending})
            live = [rid for rid in live if rid not in ending]
            k += 1
    return steps


def collect(steps, read_step) -> dict[str, dict[int, np.ndarray]]:
    """{request: {position: logits row}} from per-step arrays; `read_step(step)` -> [wanted, vocab]."""
    pos: dict[str, int] = {}
    out: dict[str, dict[int, np.ndarray]] = {}
    for rec in steps:
        rows = None
        r = 0
        for e in rec["entries"]:
            p0 = pos.get(e["id"], 0)
            for w in e["want"]:
                if rows is None:
                    rows = read_step(rec["step"])
                out.setdefault(e["id"], {})[p0 + w] = rows[r]
                r += 1
            pos[e["id"]] = p0 + len(e["tokens"])
        if rows is not None:
            assert r == rows.shape[0], f"step {rec['step']}: {rows.shape[0]} rows written, {r} wanted"
        for rid in rec["end"]:
            pos.pop(rid, None)
    return out


def run_trace_in_process(model, steps) -> dict[str, dict[int, np.ndarray]]:
    """Drive a LanguageModel the way bin/trace_run does."""
    from garlic_inference_b200 import StepEntry
    slots, results = {}, {}
    for rec in steps:
        entries = []
        for e in rec["entries"]:
            if e["id"] not in slots:
                slots[e["id"]] = model.alloc_slot()
            entries.append(StepEntry(slots[e["id"]], e["tokens"], e["want"]))
        logits = model.step(entries)
        if logits is not None:
            results[rec["step"]] = logits.float().cpu().numpy()
        for rid in rec["end"]:
            model.free_slot(slots.pop(rid))
    model.engine.check()
    return collect(steps, lambda s: results[s])


def run_trace_program(model_dir, dtype: str, steps, out_dir, max_tokens: int, vocab: int, extra_args=(),
                      env=None) -> dict[str, dict[int, np.ndarray]]:
    """Run bin/trace_run as a child process on the steps and read what it wrote."""
    out_dir = Path(out_dir)
    cmd = [sys.executable, str(REPO / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens), *extra_args]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    r = subprocess.run(cmd, input=text, capture_output=True, text=True, env=env or os.environ.copy(), timeout=900)
    assert r.returncode == 0, f"trace_run failed ({r.returncode}):\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    done = [l for l in r.stdout.splitlines() if l.startswith("done ")]
    assert [l.split()[1] for l in done] == [str(s["step"]) for s in steps], "a 'done' line per step, in order"
    return collect(steps, lambda s: np.fromfile(out_dir / f"{s}.f32", dtype="<f4").reshape(-1, vocab))


def compare(got: dict[str, dict[int, np.ndarray]], want: dict[str, np.ndarray], tol: float, what: str) -> float:
    """Every (request, position) of `got` against the plain logits; returns the worst relative error.
    On failure names the first wrong place, which is where to look (a prompt's end, the first decoded
    token, a page's edge, a slot used again)."""
    worst = 0.0
    for rid in sorted(got):
        ref = want[rid]
        scale = float(np.abs(ref).max())
        for p in sorted(got[rid]):
            row = got[rid][p]
            assert np.isfinite(row).all(), f"{what}: request {rid} position {p}: non-finite logits"
            err = float(np.abs(row - ref[p]).max()) / scale
            assert err <= tol, (f"{what}: request {rid} (length {ref.shape[0]}) first differs at position {p}: "
                                f"relative error {err:.3e} > {tol:.1e}")
            worst = max(worst, err)
    return worst


def assert_covers(got, requests) -> None:
    for rid, toks in requests.items():
        assert sorted(got.get(rid, {})) == list(range(len(toks))), f"request {rid}: not every position was returned"
