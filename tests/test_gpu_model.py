"""The engine against the plain implementation, in float32 and in bfloat16: every request alone and
whole; with the last 32 tokens one by one; in batches of unequal lengths whose shorter requests end
earlier, one batch after another in a cache too small to hold them all at once (slots and pages are
used again); long decoding; the first tokens of a sequence."""
import numpy as np
import pytest
import torch

import tiny

pytestmark = pytest.mark.gpu

LENGTHS = {
    "A": [7, 128, 33, 64, 1, 65, 100],
    "B": [5, 11, 2, 250, 97, 64, 129],
    "C": [90, 41, 40, 200, 17, 3, 130],
    "D": [300, 64, 1, 129, 700, 65, 128],
    "E": [260, 101, 100, 64, 400, 99, 129],
}
PAGE = {"A": 16, "B": 16, "C": 16, "D": 64, "E": 64}
BATCHES = [["r0", "r1", "r2"], ["r3", "r4"], ["r5", "r6"]]


def _round64(n):
    return -(-n // 64) * 64


@pytest.fixture(scope="module")
def plain_cache(model_dirs):
    made = {}

    def get(name):
        if name not in made:
            vocab = tiny.TINY[name]["cfg"]["vocab_size"]
            reqs = tiny.random_requests(vocab, LENGTHS[name], seed=ord(name))
            made[name] = (reqs, tiny.plain_logits(model_dirs(name), reqs))
        return made[name]

    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_every_cutting_agrees_with_the_plain_implementation(name, dtype, gpu_models, plain_cache):
    reqs, want = plain_cache(name)
    tol = tiny.TOL[dtype]
    # a cache that holds the largest batch and no more: later batches must reuse slots and pages
    max_tokens = max(sum(_round64(len(reqs[r])) for r in b) for b in BATCHES)
    model = gpu_models(name, dtype, max_tokens=max_tokens, page_size=PAGE[name])

    whole = tiny.run_trace_in_process(model, tiny.trace_whole(reqs))
    tiny.assert_covers(whole, reqs)
    worst = {"whole": tiny.compare(whole, want, tol, f"{name} {dtype} whole")}

    tail = tiny.run_trace_in_process(model, tiny.trace_tail_by_one(reqs, tail=32))
    tiny.assert_covers(tail, reqs)
    worst["tail"] = tiny.compare(tail, want, tol, f"{name} {dtype} last 32 one by one")

    batched = tiny.run_trace_in_process(model, tiny.trace_batched(reqs, BATCHES, prompt_frac=0.5))
    tiny.assert_covers(batched, reqs)
    worst["batched"] = tiny.compare(batched, want, tol, f"{name} {dtype} unequal batches")
    print(f"WORST {name} {dtype} " + " ".join(f"{k}={v:.3e}" for k, v in worst.items()))
    tiny.check_seen(name, dtype, max(worst.values()))

    cache = model.engine.cache
    assert cache.slots.n_free == cache.max_slots
    assert all(g.host.pool.n_free == g.host.pool.n_pages for g in cache.groups), "a page was lost"

    if dtype == "float32":
        # the float32 kernels sum in an order that depends on the position alone: the three cuttings
        # give the same bits, not merely the same numbers up to rounding
        for rid in reqs:
            for p in range(len(reqs[rid])):
                assert np.array_equal(whole[rid][p], tail[rid][p]), f"{name}: {rid} position {p}: whole vs one by one"
                assert np.array_equal(whole[rid][p], batched[rid][p]), f"{name}: {rid} position {p}: whole vs batched"


def _large_batch_requests(name, n, seed):
    """n + 8 requests of 50 to 110 tokens: a batch of n that starts together, then a batch of 8 in the same cache."""
    vocab = tiny.TINY[name]["cfg"]["vocab_size"]
    rng = np.random.default_rng(seed)
    lengths = rng.integers(50, 111, size=n + 8).tolist()
    reqs = tiny.random_requests(vocab, lengths, seed=seed + 1)
    ids = list(reqs)
    return reqs, [ids[:n], ids[n:]]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n", [12, 20, 40, 70])
@pytest.mark.parametrize("name", ["D", "E"])
def test_batches_of_many_sequences(name, n, dtype, model_dirs):
    """Batches of 12, 20, 40 and 70 sequences of unequal lengths that start together (unequal prompts in one step),
    then decode for 40 to 80 steps while the shorter ones end, then a second batch in the slots and pages the first
    gave back: the recorded steps of 16, 32, 64 and 128 rows with their padding rows, the products that take 9 to
    64 rows and more, and the decode attention that writes its output itself (256 and more (sequence, head) pairs)."""
    from garlic_inference_b200 import AutoModel
    reqs, batches = _large_batch_requests(name, n, seed=1000 + n)
    want = tiny.plain_logits(model_dirs(name), reqs)
    max_tokens = sum(_round64(len(reqs[r])) for r in batches[0])
    model = AutoModel.from_pretrained(model_dirs(name), device=0, dtype=dtype, max_tokens=max_tokens, page_size=64)
    steps = tiny.trace_batched(reqs, batches, prompt_frac=0.25)
    assert sum(1 for s in steps if len(s["entries"]) >= min(n, 9)) >= 12      # many steps at (nearly) full width
    got = tiny.run_trace_in_process(model, steps)
    tiny.assert_covers(got, reqs)
    worst = tiny.compare(got, want, tiny.TOL[dtype], f"{name} {dtype} batch of {n}")
    print(f"{name} {dtype} batch of {n}: worst relative error {worst:.3e}")
    buckets = sorted(model.engine.graphs._graphs)
    assert max(buckets) == 1 << (n - 1).bit_length(), buckets
    cache = model.engine.cache
    assert cache.slots.n_free == cache.max_slots
    assert all(g.host.pool.n_free == g.host.pool.n_pages for g in cache.groups), "a page was lost"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_batches_beyond_the_largest_recorded_size(dtype, model_dirs):
    """With the largest recorded batch size forced down to 8, a batch of 12 decodes launch by launch and smaller
    ones (as its sequences end) from recorded steps: both against the plain implementation."""
    from garlic_inference_b200 import AutoModel
    reqs, batches = _large_batch_requests("D", 12, seed=2012)
    want = tiny.plain_logits(model_dirs("D"), reqs)
    model = AutoModel.from_pretrained(model_dirs("D"), device=0, dtype=dtype, max_tokens=4096, page_size=64)
    model.engine.graphs.largest = 8
    got = tiny.run_trace_in_process(model, tiny.trace_batched(reqs, batches, prompt_frac=0.25))
    tiny.assert_covers(got, reqs)
    tiny.compare(got, want, tiny.TOL[dtype], f"D {dtype} batch of 12, recorded sizes up to 8")
    assert max(model.engine.graphs._graphs) == 8


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D", "E"])
def test_mixed_steps(name, dtype, gpu_models, model_dirs):
    """Steps that mix: request x decodes one token a step while request y's prompt arrives in two chunks of 70 and
    59 tokens, and request z's whole prompt arrives later beside both decoding."""
    vocab = tiny.TINY[name]["cfg"]["vocab_size"]
    reqs = tiny.random_requests(vocab, [90, 160, 75], seed=31)
    x, y, z = reqs["r0"], reqs["r1"], reqs["r2"]
    want = tiny.plain_logits(model_dirs(name), reqs)
    model = gpu_models(name, dtype, max_tokens=4096, page_size=64 if name in "DE" else 16)
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": x[:50], "want": list(range(50))}], "end": []},
             {"step": 1, "entries": [{"id": "r0", "tokens": [x[50]], "want": [0]},
                                     {"id": "r1", "tokens": y[:70], "want": list(range(70))}], "end": []},
             {"step": 2, "entries": [{"id": "r1", "tokens": y[70:129], "want": list(range(59))},
                                     {"id": "r0", "tokens": [x[51]], "want": [0]}], "end": []}]
    nx, ny, nz = 52, 129, 0
    while nx < len(x) or ny < len(y) or nz < len(z):
        entries = []
        if nx < len(x):
            entries.append({"id": "r0", "tokens": [x[nx]], "want": [0]})
            nx += 1
        if ny < len(y):
            entries.append({"id": "r1", "tokens": [y[ny]], "want": [0]})
            ny += 1
        if nz == 0 and nx >= 60:
            entries.append({"id": "r2", "tokens": z[:40], "want": list(range(40))})      # a prompt beside decoding rows
            nz = 40
        elif 0 < nz < len(z):
            entries.append({"id": "r2", "tokens": [z[nz]], "want": [0]})
            nz += 1
        steps.append({"step": len(steps), "entries": entries, "end": []})
    steps[-1]["end"] = ["r0", "r1", "r2"]
    got = tiny.run_trace_in_process(model, steps)
    tiny.assert_covers(got, reqs)
    tiny.compare(got, want, tiny.TOL[dtype], f"{name} {dtype} mixed steps")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_float32_is_far_closer_than_bfloat16(dtype, gpu_models, plain_cache):
    """The float32 path is a true 32-bit path: its error is orders of magnitude below bfloat16's."""
    reqs, want = plain_cache("B")
    model = gpu_models("B", dtype, max_tokens=4096, page_size=16)
    got = tiny.run_trace_in_process(model, tiny.trace_whole({"r3": reqs["r3"]}))
    worst = tiny.compare(got, want, tiny.TOL[dtype], f"B {dtype}")
    if dtype == "float32":
        assert worst < 2e-5
    else:
        assert worst > 2e-5, "bfloat16 cannot be this exact: is the float32 path running instead?"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,n_prompt,n_total", [("F", 10, 640), ("C", 3, 300)])
def test_long_decoding(name, n_prompt, n_total, dtype, gpu_models, model_dirs):
    vocab = tiny.TINY[name]["cfg"]["vocab_size"]
    reqs = tiny.random_requests(vocab, [n_total], seed=11)
    want = tiny.plain_logits(model_dirs(name), reqs)
    model = gpu_models(name, dtype, max_tokens=4096, page_size=16)
    steps = tiny.trace_tail_by_one(reqs, tail=n_total - n_prompt)
    got = tiny.run_trace_in_process(model, steps)
    tiny.assert_covers(got, reqs)
    tiny.compare(got, want, tiny.TOL[dtype], f"{name} {dtype} decoding {n_total - n_prompt} tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_first_tokens_of_a_sequence(name, dtype, gpu_models, model_dirs):
    vocab = tiny.TINY[name]["cfg"]["vocab_size"]
    reqs = tiny.random_requests(vocab, [1, 2, 3, 1], seed=12)
    want = tiny.plain_logits(model_dirs(name), reqs)
    model = gpu_models(name, dtype, max_tokens=4096, page_size=16)
    for steps in (tiny.trace_whole(reqs), tiny.trace_tail_by_one(reqs, tail=32),
                  tiny.trace_batched(reqs, [["r0", "r1", "r2", "r3"]], prompt_frac=0.0)):
        got = tiny.run_trace_in_process(model, steps)
        tiny.assert_covers(got, reqs)
        tiny.compare(got, want, tiny.TOL[dtype], f"{name} {dtype} first tokens")


def test_padding_rows_change_nothing(gpu_models, plain_cache):
    """Rows with slot -1 may ride along in a step (a padded batch): the others' logits keep their bits."""
    from garlic_inference_b200.parts import StepContext
    reqs, _ = plain_cache("A")
    model = gpu_models("A", "float32", max_tokens=4096, page_size=16)
    eng = model.engine
    toks = reqs["r2"]

    def run(pad):
        s = eng.alloc_slot()
        n = len(toks)
        eng.cache.prepare([s], [n])
        t = torch.tensor(toks + [0] * pad, dtype=torch.int32, device="cuda")
        pos = torch.tensor(list(range(n)) + [0] * pad, dtype=torch.int32, device="cuda")
        slot = torch.tensor([s] * n + [-1] * pad, dtype=torch.int32, device="cuda")
        ctx = StepContext(n_tokens=n + pad, tokens=t, tok_pos=pos, tok_slot=slot, seq_slots=[s], seq_starts=[0],
                          seq_lens=[n], seq_past=[0], max_kv_len=n, status=eng.cache.status)
        rows = torch.arange(n, dtype=torch.int32, device="cuda")
        out = model.model.forward(ctx, eng.cache, rows).cpu()
        eng.cache.commit([s], [n])
        eng.free_slot(s)
        return out

    plain_run, padded = run(0), run(5)
    assert torch.equal(plain_run, padded)
    eng.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_recorded_decode_steps_equal_launched_ones(dtype, model_dirs, plain_cache):
    """Decode steps replayed from CUDA graphs (the default) against the same steps launched kernel by
    kernel: same bits in float32; batches of 1, 2, 3 (padded to 4) and 5 (padded to 8) sequences."""
    from garlic_inference_b200 import AutoModel
    reqs, want = plain_cache("C")
    steps = tiny.trace_batched(reqs, [["r0"], ["r1", "r2"], ["r3", "r4", "r5"], ["r0", "r1", "r2", "r3", "r6"]],
                               prompt_frac=0.3)
    got = {}
    for graphs in (True, False):
        model = AutoModel.from_pretrained(model_dirs("C"), device=0, dtype=dtype, max_tokens=1024, page_size=16,
                                          use_graphs=graphs)
        assert (model.engine.graphs is not None) == graphs
        got[graphs] = tiny.run_trace_in_process(model, steps)
        tiny.compare(got[graphs], want, tiny.TOL[dtype], f"C {dtype} graphs={graphs}")
        if graphs:
            assert sorted(model.engine.graphs._graphs) == [1, 2, 4, 8]
    if dtype == "float32":
        for rid in got[True]:
            for p in got[True][rid]:
                assert np.array_equal(got[True][rid][p], got[False][rid][p]), f"{rid} position {p}"


def test_step_errors_come_before_any_launch(gpu_models):
    from garlic_inference_b200.cache import CacheError
    from garlic_inference_b200.engine import StepEntry, StepError
    model = gpu_models("A", "float32", max_tokens=128, page_size=16)
    s = model.alloc_slot()
    try:
        with pytest.raises(StepError, match="outside the vocabulary"):
            model.step([StepEntry(s, [1, 512], [0])])
        with pytest.raises(StepError, match="want index"):
            model.step([StepEntry(s, [1, 2], [2])])
        with pytest.raises(StepError, match="no tokens"):
            model.step([StepEntry(s, [], [])])
        with pytest.raises(CacheError, match="limit is 128"):
            model.step([StepEntry(s, [1] * 129, [])])
        assert model.engine.cache.length(s) == 0
        assert model.step([StepEntry(s, [1, 2, 3], [])]) is None          # nothing wanted: nothing returned
        assert model.engine.cache.length(s) == 3
        out = model.step([StepEntry(s, [4], [0])])
        assert out.shape == (1, 512) and out.dtype == torch.float32
    finally:
        model.free_slot(s)


def test_tcgen05_products_in_the_model(model_dirs, plain_cache, monkeypatch):
    """The same cuttings with this package's tcgen05 kernel taking every product of more than 8 rows
    (the library product is the default there)."""
    from garlic_inference_b200 import AutoModel
    import sys
    monkeypatch.setattr(sys.modules["garlic_inference_b200.ops.linear"], "LARGE_GEMM", "tcgen05")
    reqs, want = plain_cache("D")
    model = AutoModel.from_pretrained(model_dirs("D"), device=0, dtype="bfloat16", max_tokens=2048, page_size=64)
    for steps in (tiny.trace_whole(reqs), tiny.trace_batched(reqs, BATCHES, prompt_frac=0.5)):
        got = tiny.run_trace_in_process(model, steps)
        tiny.assert_covers(got, reqs)
        tiny.compare(got, want, tiny.TOL["bfloat16"], "D bfloat16 with tcgen05 products")


def test_streamk_products_in_the_model(model_dirs, plain_cache, monkeypatch):
    """Decode steps (recorded and replayed) with the stream-K tcgen05 kernel taking every product of 1 to 8
    rows, which by default it does only for weights of 256 MB and more."""
    import sys
    from garlic_inference_b200 import AutoModel
    monkeypatch.setattr(sys.modules["garlic_inference_b200.ops.linear"], "STREAMK_MIN_BYTES", 1)
    monkeypatch.setattr(sys.modules["garlic_inference_b200.ops.linear"], "STREAMK_MIN_BYTES_WIDE", 1)
    reqs, want = plain_cache("D")
    model = AutoModel.from_pretrained(model_dirs("D"), device=0, dtype="bfloat16", max_tokens=2048, page_size=64)
    for steps in (tiny.trace_tail_by_one(reqs, tail=32), tiny.trace_batched(reqs, BATCHES, prompt_frac=0.5)):
        got = tiny.run_trace_in_process(model, steps)
        tiny.assert_covers(got, reqs)
        tiny.compare(got, want, tiny.TOL["bfloat16"], "D bfloat16 with stream-K products")


def test_gemv_products_in_the_model(model_dirs, plain_cache, monkeypatch):
    """Steps of one sequence with the gemv kernels (plain and with the SwiGLU in it) taking every one-row product,
    which by default the skinny and stream-K kernels take."""
    import sys
    from garlic_inference_b200 import AutoModel
    monkeypatch.setattr(sys.modules["garlic_inference_b200.ops.linear"], "GEMV_MAX_ROWS", 1)
    reqs, want = plain_cache("D")
    model = AutoModel.from_pretrained(model_dirs("D"), device=0, dtype="bfloat16", max_tokens=2048, page_size=64)
    got = tiny.run_trace_in_process(model, tiny.trace_tail_by_one(reqs, tail=32))
    tiny.assert_covers(got, reqs)
    tiny.compare(got, want, tiny.TOL["bfloat16"], "D bfloat16 with gemv products")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_step_by_step_against_the_plain_model_with_the_same_interface(dtype, gpu_models, model_dirs):
    """The engine and the plain model behind the same stepping interface (tests/plain_stepper.py) replay one
    schedule side by side: unequal prompts in one step, single tokens, a request that ends early, a slot used
    again, a mixed step.  Every step's logits are compared as the step returns them."""
    from plain_stepper import PlainStepper, first_step_that_differs
    vocab = tiny.TINY["C"]["cfg"]["vocab_size"]
    reqs = tiny.random_requests(vocab, [60, 23, 90, 41], seed=77)
    steps = tiny.trace_batched(reqs, [["r0", "r1", "r2"], ["r3", "r1"]], prompt_frac=0.6)
    model = gpu_models("C", dtype, max_tokens=4096, page_size=16)
    bad = first_step_that_differs(model, PlainStepper(model_dirs("C")), steps, tiny.TOL[dtype])
    assert bad is None, f"step {bad[0]} is the first that differs (relative error {bad[1]:.3e})"
