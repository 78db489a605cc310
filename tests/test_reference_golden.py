"""The plain implementation (CPU) and the engine (GPU) against logits that upstream's own dense Qwen3 code
produced on a B200 (tests/golden/reference_*.npz, made by tests/golden/make_reference_golden.py).

Upstream computes in bfloat16 with a rounding after every operation; the bound is the one the other
bfloat16 comparisons use, relative to the largest logit.  What these files pin on upstream's own output and
no formula in upstream's sources states: query head h reads key/value head h // group, and the causal mask
aligned to the bottom right when new tokens attend to a filled cache (both are left to a library there,
src/src-cuda/attention/fattn.cu:74-86)."""
from pathlib import Path

import numpy as np
import pytest
import torch

import tiny

GOLDEN = Path(__file__).resolve().parent / "golden"
NAMES = [n for n in ("A", "G") if (GOLDEN / f"reference_{n}.npz").is_file()]
# worst error seen when the files were made, relative to the largest logit: plain float32 against upstream
SEEN = {"A": 3.5e-3, "G": 7.1e-3}


def load(name):
    z = np.load(GOLDEN / f"reference_{name}.npz")
    logits = (z["logits"].astype(np.uint32) << 16).view(np.float32)
    return z["ids"], logits


def test_the_golden_files_are_there():
    assert NAMES == ["A", "G"], "tests/golden lacks upstream's logits (make_reference_golden.py writes them)"


@pytest.mark.parametrize("name", NAMES)
def test_plain_implementation_against_upstreams_own_logits(name, model_dirs):
    ids, ref = load(name)
    requests = {f"b{b}": ids[b].tolist() for b in range(ids.shape[0])}
    want = tiny.plain_logits(model_dirs(name), requests)
    worst = 0.0
    for b in range(ids.shape[0]):
        scale = float(np.abs(want[f"b{b}"]).max())
        err = np.abs(ref[b] - want[f"b{b}"]).max(axis=1) / scale
        assert err.max() <= tiny.TOL["bfloat16"], f"{name}: sequence {b} first differs at position {int(err.argmax())}"
        worst = max(worst, float(err.max()))
        # the greedy token is the same wherever the plain top-2 margin is beyond the rounding
        top2 = np.sort(want[f"b{b}"], axis=1)[:, -2:]
        sure = (top2[:, 1] - top2[:, 0]) > 2 * tiny.TOL["bfloat16"] * scale
        assert (ref[b].argmax(1)[sure] == want[f"b{b}"].argmax(1)[sure]).all()
    print(f"plain vs upstream {name}: worst relative error {worst:.3e}")
    assert worst <= 2 * SEEN[name], f"{name}: {worst:.3e} is more than twice the error seen when the files were made"


@pytest.mark.parametrize("name", NAMES)
def test_the_comparison_catches_a_wrong_reading(name, model_dirs, monkeypatch):
    """Query head h reading key/value head h % n_kv instead of h // group, or the rotation with its sign
    turned: either moves the logits away from upstream's by far more than the bound."""
    import math
    import plain_qwen3 as plain
    ids, ref = load(name)
    requests = {"b0": ids[0].tolist()}

    def worst():
        want = tiny.plain_logits(model_dirs(name), requests)["b0"]
        return float(np.abs(ref[0] - want).max() / np.abs(want).max())

    def kv_head_modulo(q, k, v, window=None):
        S, n_q, d = q.shape
        n_kv = k.shape[1]
        out = torch.empty_like(q)
        pos = torch.arange(S)
        allowed = pos[None, :] <= pos[:, None]
        for h in range(n_q):
            s = ((q[:, h, :] @ k[:, h % n_kv, :].T) / math.sqrt(d)).masked_fill(~allowed, float("-inf"))
            out[:, h, :] = torch.softmax(s, dim=-1) @ v[:, h % n_kv, :]
        return out

    def rotation_turned(x, positions, theta):
        d = x.shape[-1]
        ang = plain.rope_angles(positions, d, theta, torch.float64)
        cos, sin = ang.cos().to(x.dtype)[:, None, :], ang.sin().to(x.dtype)[:, None, :]
        x1, x2 = x[..., : d // 2], x[..., d // 2:]
        return torch.cat([x1 * cos + x2 * sin, x2 * cos - x1 * sin], dim=-1)

    assert worst() <= tiny.TOL["bfloat16"]
    with monkeypatch.context() as m:
        m.setattr(plain, "attention_scores", kv_head_modulo)
        assert worst() > 5 * tiny.TOL["bfloat16"]
    with monkeypatch.context() as m:
        m.setattr(plain, "apply_rope", rotation_turned)
        assert worst() > 5 * tiny.TOL["bfloat16"]


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_engine_bfloat16_against_upstreams_own_logits(name, gpu_models):
    """The same schedule upstream ran: the prompts of a batch in one step, then one given token each per step."""
    ids, ref = load(name)
    model = gpu_models(name, "bfloat16", 4096, 64 if name == "G" else 16)
    prompt = 40
    requests = {f"b{b}": ids[b].tolist() for b in range(ids.shape[0])}
    steps = tiny.trace_batched(requests, [list(requests)], prompt_frac=prompt / ids.shape[1])
    got = tiny.run_trace_in_process(model, steps)
    tiny.assert_covers(got, requests)
    worst = tiny.compare(got, {f"b{b}": ref[b] for b in range(ids.shape[0])}, tiny.TOL["bfloat16"],
                         f"engine bfloat16 vs upstream {name}")
    print(f"engine vs upstream {name}: worst relative error {worst:.3e}")
    assert worst <= 2 * SEEN[name]
