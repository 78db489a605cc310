"""Generation through the Python entry point and the command line, against the plain greedy loop."""
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import tiny

pytestmark = pytest.mark.gpu


def _cut(tokens, stop):
    return tokens[:tokens.index(stop) + 1] if stop in tokens else tokens


def _check_greedy(name, model_dir, prompts, got, n_new, dtype, stop_ids=()):
    """Every generated token is the plain implementation's choice; in bfloat16 a different token is
    accepted only where the plain logits of the two lie within the bfloat16 tolerance, and the
    comparison of that request stops there (the continuations differ from then on)."""
    cfg, w = plain.read_model_dir(model_dir)
    for prompt, new in zip(prompts, got):
        ids = list(prompt)
        for k, tok in enumerate(new):
            logits = plain.forward(cfg, w, ids)[-1]
            best = int(logits.argmax())
            if tok != best:
                gap = float(logits[best] - logits[tok]) / float(logits.abs().max())
                assert dtype == "bfloat16" and gap <= tiny.TOL["bfloat16"], (
                    f"{name} {dtype}: prompt of {len(prompt)}, new token {k}: engine chose {tok}, plain {best} "
                    f"(relative gap {gap:.2e})")
                break
            ids.append(tok)
            if tok in stop_ids:
                assert k == len(new) - 1, "nothing is generated after a stop token"
                break
        else:
            assert len(new) == n_new or len(prompt) + len(new) >= cfg["max_position_embeddings"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_matches_the_plain_loop(name, dtype, gpu_models, model_dirs):
    vocab = tiny.TINY[name]["cfg"]["vocab_size"]
    prompts = list(tiny.random_requests(vocab, [9, 1, 30, 17, 5], seed=41).values())
    model = gpu_models(name, dtype, max_tokens=256, page_size=16)        # 4 slots: two batches, slots reused
    got = model.generate(prompts, max_new_tokens=12)
    assert model.last_stats.batches == 2 and model.last_stats.new_tokens == sum(len(g) for g in got)
    _check_greedy(name, model_dirs(name), prompts, got, 12, dtype)
    again = model.generate(prompts[::-1], max_new_tokens=12)
    if dtype == "float32":
        assert again[::-1] == got, "a request's tokens do not depend on its batch"


def test_stop_tokens_and_position_limit(gpu_models, model_dirs):
    model = gpu_models("A", "float32", max_tokens=512, page_size=16)
    prompts = list(tiny.random_requests(512, [6, 20, 120], seed=42).values())
    free_run = model.generate(prompts, max_new_tokens=10)
    stop = free_run[0][3]
    assert len(free_run[2]) == 8                                         # 120 + 8 = 128 positions: the model's limit
    got = model.generate(prompts, max_new_tokens=10, stop_token_ids=[stop])
    assert got == [_cut(f, stop) for f in free_run] and len(got[0]) <= 4
    _check_greedy("A", model_dirs("A"), prompts, got, 10, "float32", stop_ids=(stop,))
    assert model.last_stats.batch_sizes[0] == 3 and model.last_stats.batch_sizes[-1] < 3
    cache = model.engine.cache
    assert cache.slots.n_free == cache.max_slots


def test_temperature_sampling_is_seeded_and_independent_of_the_batch(gpu_models):
    model = gpu_models("B", "float32", max_tokens=1024, page_size=16)
    prompts = list(tiny.random_requests(1000, [8, 3, 21], seed=43).values())
    a = model.generate(prompts, max_new_tokens=16, temperature=0.9, seed=7)
    b = model.generate(prompts, max_new_tokens=16, temperature=0.9, seed=7)
    c = model.generate(prompts, max_new_tokens=16, temperature=0.9, seed=8)
    greedy = model.generate(prompts, max_new_tokens=16)
    assert a == b and a != c and a != greedy
    # the same requests run one at a time draw the same tokens: request i keeps its number only if
    # it is given at the same place, so pad the list with the others' places
    alone = model.generate(prompts, max_new_tokens=16, temperature=0.9, seed=7, max_batch=1)
    assert alone == a
    assert all(0 <= t < 1000 for g in a for t in g)


def test_command_line(model_dirs):
    cmd = [sys.executable, str(tiny.REPO / "bin" / "runner"), str(model_dirs("A")), "--max-new-tokens", "5",
           "--dtype", "float32"]
    r = subprocess.run(cmd, input="1 2 3\n40,41\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    lines = r.stdout.strip().splitlines()
    assert len(lines) == 5 and lines[2].startswith("Time: ") and lines[3].startswith("Tok/s: ")
    cfg, w = plain.read_model_dir(model_dirs("A"))
    assert [int(t) for t in lines[0].split()] == plain.greedy(cfg, w, [1, 2, 3], 5)
    assert [int(t) for t in lines[1].split()] == plain.greedy(cfg, w, [40, 41], 5)
    r2 = subprocess.run(cmd + ["--prompt-ids", "1,2,3", "--stop-ids", lines[0].split()[1]], capture_output=True,
                        text=True, timeout=600)
    assert r2.returncode == 0 and r2.stdout.splitlines()[0].split() == _cut(lines[0].split(), lines[0].split()[1])


def test_command_line_prompt_file_and_random_weights(model_dirs, tmp_path):
    """--prompt-file reads one prompt a line; --random-weights needs a config.json alone and gives the same
    ids from run to run for one --weights-seed."""
    prompts = tmp_path / "prompts.txt"
    prompts.write_text("1 2 3\n\n40,41\n")
    cmd = [sys.executable, str(tiny.REPO / "bin" / "runner"), str(model_dirs("A")), "--max-new-tokens", "4",
           "--dtype", "float32", "--prompt-file", str(prompts)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    cfg, w = plain.read_model_dir(model_dirs("A"))
    lines = r.stdout.strip().splitlines()
    assert [int(t) for t in lines[0].split()] == plain.greedy(cfg, w, [1, 2, 3], 4)
    assert [int(t) for t in lines[1].split()] == plain.greedy(cfg, w, [40, 41], 4)
    only_config = tmp_path / "cfg"
    only_config.mkdir()
    (only_config / "config.json").write_text((model_dirs("B") / "config.json").read_text())
    cmd = [sys.executable, str(tiny.REPO / "bin" / "runner"), str(only_config), "--random-weights", "--weights-seed", "5",
           "--max-new-tokens", "6", "--prompt-ids", "9,8,7"]
    runs = [subprocess.run(cmd, capture_output=True, text=True, timeout=600) for _ in range(2)]
    assert all(x.returncode == 0 for x in runs), runs[0].stderr[-3000:]
    first = runs[0].stdout.splitlines()[0].split()
    assert len(first) == 6 and first == runs[1].stdout.splitlines()[0].split()


def test_smoke_entry():
    sys.path.insert(0, str(tiny.REPO))
    import __graft_entry__ as entry
    entry.smoke()


def test_timeline_of_a_recorded_step(model_dirs):
    """`python -m garlic_inference_b200.engine.timeline` on a tiny model: the second build (with marks in the
    kernels) compiles, every kernel of the replayed step leaves both marks in launch order, and the repeating
    layer is found."""
    cmd = [sys.executable, "-m", "garlic_inference_b200.engine.timeline", "--config",
           str(model_dirs("D") / "config.json"), "--layers", "5", "--batch", "3", "--cached", "70"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=str(tiny.REPO))
    assert r.returncode == 0, r.stderr[-3000:]
    head = r.stdout.splitlines()[0]
    assert "kernels" in head and "a layer is 9 kernels" in head, r.stdout[:2000]
    assert "a layer:" in r.stdout


def test_command_line_print_logits_and_max_slots(model_dirs):
    """--print-logits N prints the N largest logits at each prompt's last position before generating;
    --max-slots 1 lets one request live at a time, so two prompts run as two batches with the same ids."""
    cmd = [sys.executable, str(tiny.REPO / "bin" / "runner"), str(model_dirs("A")), "--max-new-tokens", "4",
           "--dtype", "float32", "--prompt-ids", "1,2,3", "--prompt-ids", "40,41", "--print-logits", "3",
           "--max-slots", "1", "--max-tokens", "128"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    lines = r.stdout.strip().splitlines()
    cfg, w = plain.read_model_dir(model_dirs("A"))
    for i, prompt in enumerate(([1, 2, 3], [40, 41])):
        assert lines[i].startswith(f"Logits {i}: ")
        pairs = [p.split(":") for p in lines[i].split(": ", 1)[1].split()]
        want = plain.forward(cfg, w, prompt)[-1]
        top = want.topk(3)
        assert [int(t) for t, _ in pairs] == top.indices.tolist()
        assert all(abs(float(v) - float(x)) < 1e-4 * float(want.abs().max()) for (_, v), x in zip(pairs, top.values))
        assert [int(t) for t in lines[2 + i].split()] == plain.greedy(cfg, w, prompt, 4)
