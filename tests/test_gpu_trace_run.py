"""bin/trace_run as a user runs it: a child process fed steps on standard input, whose <step>.f32
files are compared with the plain implementation, in float32 and in bfloat16, for whole requests,
the last 32 tokens one by one, and unequal batches in a cache that makes slots be used again."""
import json
import subprocess
import sys

import numpy as np
import pytest

import tiny

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C"])
def test_trace_run_all_cuttings(name, dtype, model_dirs, tmp_path):
    vocab = tiny.TINY[name]["cfg"]["vocab_size"]
    reqs = tiny.random_requests(vocab, [70, 5, 130, 33, 64], seed=31)
    want = tiny.plain_logits(model_dirs(name), reqs)
    batches = [["r0", "r1", "r2"], ["r3", "r4"]]
    steps = tiny.trace_whole(reqs)
    off = len(steps)
    for more in (tiny.trace_tail_by_one(reqs, tail=32), tiny.trace_batched(reqs, batches)):
        for s in more:
            steps.append({**s, "step": s["step"] + off})
        off = len(steps)
    # one process runs the three cuttings one after another: 128 + 64 + 192 tokens is the most that is live
    out = tmp_path / "out"
    results = tiny.run_trace_program(model_dirs(name), dtype, steps, out, max_tokens=384, vocab=vocab)
    # `collect` keeps the last logits seen for a (request, position); check each cutting on its own too
    tiny.assert_covers(results, reqs)
    tiny.compare(results, want, tiny.TOL[dtype], f"trace_run {name} {dtype} (last cutting)")
    n_whole = len(tiny.trace_whole(reqs))
    n_tail = len(tiny.trace_tail_by_one(reqs, tail=32))
    for label, lo, hi, sub in (("whole", 0, n_whole, tiny.trace_whole(reqs)),
                               ("one by one", n_whole, n_whole + n_tail, tiny.trace_tail_by_one(reqs, tail=32))):
        part = tiny.collect(sub, lambda s, lo=lo: np.fromfile(out / f"{s + lo}.f32", dtype="<f4").reshape(-1, vocab))
        tiny.assert_covers(part, reqs)
        tiny.compare(part, want, tiny.TOL[dtype], f"trace_run {name} {dtype} {label}")


def test_trace_run_writes_nothing_for_steps_without_wants_and_rejects_bad_input(model_dirs, tmp_path):
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [4], "want": [0]}], "end": ["a"]},
             {"step": 2, "entries": [], "end": []}]
    out = tmp_path / "o"
    got = tiny.run_trace_program(model_dirs("A"), "float32", steps, out, max_tokens=64, vocab=512)
    assert sorted(p.name for p in out.iterdir()) == ["1.f32"]
    assert (out / "1.f32").stat().st_size == 512 * 4 and sorted(got["a"]) == [3]
    bad = subprocess.run([sys.executable, str(tiny.REPO / "bin" / "trace_run"), "--model", str(model_dirs("A")),
                          "--dtype", "float32", "--out", str(tmp_path / "o2"), "--max-tokens", "64"],
                         input=json.dumps({"step": 0, "entries": [{"id": "a", "tokens": [1] * 65, "want": []}],
                                           "end": []}) + "\n", capture_output=True, text=True, timeout=600)
    assert bad.returncode != 0 and "done 0" not in bad.stdout
    assert "positions" in bad.stderr or "cache" in bad.stderr
