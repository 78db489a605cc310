#!/usr/bin/env python3
"""Logits of upstream's own dense Qwen3 code on tiny random models, kept beside the tests.

Upstream's model code is C++/CUDA without a CPU path, so it cannot run where the CPU tests run.  On a
B200 it can: `baseline/build_reference.py` compiles upstream's unmodified dense-path sources for sm_100a
with a small driver (`baseline/reference_driver.cpp`).  This script runs that program on tiny tied
models (upstream always ties the head, src/models/qwen3/qwen3.cpp:58) in bfloat16 (upstream has no
float32 path) and stores what it printed:

    tests/golden/reference_<config>.npz
        ids     int32  [batch, prompt + steps]   the tokens fed (prompt, then one given token a step)
        logits  uint16 [batch, prompt + steps, vocab]   upstream's bfloat16 logits, as their bit patterns

The model folders are written by `tiny.write_model`, whose values depend on (seed, tensor name, index)
alone, so the tests rebuild the same weights anywhere.  `tests/test_reference_golden.py` compares the
plain implementation (CPU) and the engine (GPU) with these files.

    python tests/golden/make_reference_golden.py        # on a machine with a B200, after the build
"""
from __future__ import annotations

import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path[:0] = [str(HERE.parent), str(REPO)]

CONFIGS = ("A", "G")
BATCH, PROMPT, STEPS = 2, 40, 8        # the prompt crosses upstream's 32-token cache pages


def main() -> int:
    import tiny
    runner = REPO / "baseline" / "_ref" / "bin" / "reference_runner"
    if not runner.is_file():
        print(f"{runner} is missing: run baseline/build_reference.py first", file=sys.stderr)
        return 2
    for name in CONFIGS:
        vocab = tiny.TINY[name]["cfg"]["vocab_size"]
        ids = np.random.default_rng(100 + ord(name)).integers(0, vocab, size=(BATCH, PROMPT + STEPS)).astype(np.uint32)
        with tempfile.TemporaryDirectory() as tmp:
            folder = tiny.write_model(name, Path(tmp) / "model")
            ids.tofile(Path(tmp) / "ids.bin")
            cmd = [str(runner), str(folder), "--batch", str(BATCH), "--prompt-len", str(PROMPT), "--steps", str(STEPS),
                   "--warmup", "0", "--ids", str(Path(tmp) / "ids.bin"), "--dump", str(Path(tmp) / "logits.bin")]
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
            print(name, r.returncode, r.stdout.strip(), r.stderr.strip()[-2000:], flush=True)
            if r.returncode != 0:
                return 1
            flat = np.fromfile(Path(tmp) / "logits.bin", dtype="<f4")
        # the dump holds the prompt step [batch, prompt, vocab], then one [batch, 1, vocab] block per decode step
        head = flat[:BATCH * PROMPT * vocab].reshape(BATCH, PROMPT, vocab)
        tail = flat[BATCH * PROMPT * vocab:].reshape(STEPS, BATCH, vocab).transpose(1, 0, 2)
        logits = np.concatenate([head, tail], axis=1)
        bits = (logits.view(np.uint32) >> 16).astype(np.uint16)
        assert ((bits.astype(np.uint32) << 16).view(np.float32) == logits).all(), "the dump was not bfloat16 values"
        np.savez_compressed(HERE / f"reference_{name}.npz", ids=ids.astype(np.int32), logits=bits)
        print(f"wrote reference_{name}.npz: max |logit| {np.abs(logits).max():.3f}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
