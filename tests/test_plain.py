"""The plain implementation checked against hand-computed values and its own invariants (CPU)."""
import pytest
import math

import numpy as np
import torch

import plain_qwen3 as plain
import tiny


def test_rms_norm_and_silu_by_hand():
    x = torch.tensor([[3.0, -4.0]])
    w = torch.tensor([2.0, 0.5])
    inv = 1.0 / math.sqrt((9 + 16) / 2 + 1e-3)
    assert torch.allclose(plain.rms_norm(x, w, 1e-3), torch.tensor([[3 * inv * 2, -4 * inv * 0.5]]), atol=1e-6)
    assert float(plain.silu(torch.tensor(0.0))) == 0.0
    assert abs(float(plain.silu(torch.tensor(2.0))) - 2 / (1 + math.exp(-2))) < 1e-6


def test_rotation_is_relative_and_keeps_position_zero():
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, 32, generator=g), torch.randn(1, 1, 32, generator=g)
    assert torch.equal(plain.apply_rope(q, torch.tensor([0]), 1e4), q)

    def score(m, n):
        return float((plain.apply_rope(q.double(), torch.tensor([m]), 1e4)
                      * plain.apply_rope(k.double(), torch.tensor([n]), 1e4)).sum())

    assert abs(score(5, 3) - score(105, 103)) < 1e-9 and abs(score(5, 3) - score(6, 3)) > 1e-6
    # rotate-half pairs (i, i + d/2): with a single non-zero pair only that pair moves
    x = torch.zeros(1, 1, 8, dtype=torch.float64)
    x[..., 1] = 1.0
    y = plain.apply_rope(x, torch.tensor([3]), 100.0)
    ang = 3 * 100.0 ** (-2 * 1 / 8)
    assert torch.allclose(y[0, 0], torch.tensor([0, math.cos(ang), 0, 0, 0, math.sin(ang), 0, 0], dtype=torch.float64))


def test_attention_masks_groups_and_window():
    g = torch.Generator().manual_seed(1)
    S, n_q, n_kv, d = 9, 6, 2, 8
    q, k, v = (torch.randn(S, n, d, generator=g, dtype=torch.float64) for n in (n_q, n_kv, n_kv))
    out = plain.attention_scores(q, k, v)
    assert torch.allclose(out[0], v[0].repeat_interleave(3, dim=0))            # the first query sees one key
    rep = plain.attention_scores(q, k.repeat_interleave(3, dim=1), v.repeat_interleave(3, dim=1))
    assert torch.allclose(out, rep)                                            # head h reads kv head h // 3
    assert torch.allclose(plain.attention_scores(q, k, v, window=S), out)
    assert torch.allclose(plain.attention_scores(q, k, v, window=1), v.repeat_interleave(3, dim=1))
    w3 = plain.attention_scores(q, k, v, window=3)
    i, h = 7, 4
    s = (q[i, h] @ k[5:8, h // 3].T) / math.sqrt(d)
    assert torch.allclose(w3[i, h], torch.softmax(s, -1) @ v[5:8, h // 3])      # keys 5, 6, 7 for query 7


def test_whole_model_is_causal_and_stable_in_precision(tmp_path):
    for name in tiny.TINY:
        cfg, w = plain.read_model_dir(tiny.write_model(name, tmp_path / name))
        ids = np.random.default_rng(3).integers(0, cfg["vocab_size"], size=60).tolist()
        full = plain.forward(cfg, w, ids)
        assert full.shape == (60, cfg["vocab_size"]) and torch.isfinite(full).all()
        part = plain.forward(cfg, w, ids[:23])
        assert torch.allclose(full[:23], part, atol=1e-5 * float(full.abs().max()))
        f64 = plain.forward(cfg, w, ids, torch.float64)
        assert float((full.double() - f64).abs().max()) < 2e-5 * float(f64.abs().max())


def test_window_layers_change_the_result_only_beyond_the_window(tmp_path):
    cfg, w = plain.read_model_dir(tiny.write_model("C", tmp_path / "C"))
    assert plain.layer_windows(cfg) == [None, 40, 40, None]
    ids = np.random.default_rng(4).integers(0, cfg["vocab_size"], size=70).tolist()
    windowed = plain.forward(cfg, w, ids)
    nowin = plain.forward({**cfg, "layer_types": None, "sliding_window": None}, w, ids)
    assert torch.allclose(windowed[:40], nowin[:40], atol=1e-6)
    assert float((windowed[45:] - nowin[45:]).abs().max()) > 1e-4


def test_tied_and_separate_heads(tmp_path):
    cfg, w = plain.read_model_dir(tiny.write_model("A", tmp_path / "A"))
    assert cfg["tie_word_embeddings"] and "lm_head.weight" not in w
    h = torch.randn(3, cfg["hidden_size"])
    assert torch.equal(plain.output_head(h, w, cfg),
                       plain.rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"]) @ w["model.embed_tokens.weight"].T)


def test_greedy_matches_forward(tmp_path):
    cfg, w = plain.read_model_dir(tiny.write_model("B", tmp_path / "B"))
    new = plain.greedy(cfg, w, [5, 6, 7], 4)
    assert len(new) == 4
    assert new[1] == int(plain.forward(cfg, w, [5, 6, 7, new[0]])[-1].argmax())
    assert plain.greedy(cfg, w, [5, 6, 7], 4, stop_ids=(new[1],)) == new[:2]


def test_the_plain_model_behind_the_stepping_interface_replays_every_cutting(tmp_path):
    """`PlainStepper` (alloc_slot / step / free_slot, no cache) replays the three cuttings the engine is tested with;
    every (request, position) equals the whole-sequence logits.  This also checks the trace builders and `collect`
    themselves, on the CPU."""
    from plain_stepper import PlainStepper
    d = tiny.write_model("A", tmp_path / "A")
    reqs = tiny.random_requests(512, [9, 40, 3, 17], seed=5)
    want = tiny.plain_logits(d, reqs)
    stepper = PlainStepper(d)
    for steps in (tiny.trace_whole(reqs), tiny.trace_tail_by_one(reqs, tail=8),
                  tiny.trace_batched(reqs, [["r0", "r1"], ["r2", "r3"]], prompt_frac=0.4)):
        got = tiny.run_trace_in_process(stepper, steps)
        tiny.assert_covers(got, reqs)
        assert tiny.compare(got, want, 1e-6, "plain stepper") < 1e-6
        assert stepper.tokens == {}, "a slot was not given back"
    s = stepper.alloc_slot()
    stepper.free_slot(s)
    with pytest.raises(KeyError):
        stepper.free_slot(s)
