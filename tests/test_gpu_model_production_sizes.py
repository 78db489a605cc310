"""One layer at the sizes of the benchmark model and of its two larger siblings (Qwen3-8B: hidden 4096, 32 query
and 8 key/value heads of 128, feed-forward 12288; Qwen3-14B: hidden 5120, 40 heads, feed-forward 17408; Qwen3-32B:
hidden 5120, 64 heads, so that heads x head size is not the hidden size, feed-forward 25600), the vocabulary cut
to 2,048 so that the plain implementation stays quick, against the plain implementation: the kernels run at the
shapes they are tuned for (cluster split-K products, tcgen05 attention, the gate/up product with the SwiGLU in
its epilogue from 512 rows on) and at widths that are no power of two."""
import pytest
import torch

import tiny

pytestmark = pytest.mark.gpu

COMMON = dict(num_hidden_layers=1, num_key_value_heads=8, head_dim=128, vocab_size=2048, rope_theta=1e6,
              rms_norm_eps=1e-6, max_position_embeddings=1024, tie_word_embeddings=False)
SIZES = {
    "8B": dict(hidden_size=4096, num_attention_heads=32, intermediate_size=12288),
    "14B": dict(hidden_size=5120, num_attention_heads=40, intermediate_size=17408),
    "32B": dict(hidden_size=5120, num_attention_heads=64, intermediate_size=25600),
}
LENGTHS = [600, 130, 64, 33]


@pytest.fixture(scope="module", params=list(SIZES))
def big_layer(request, tmp_path_factory):
    from garlic_inference_b200 import Qwen3Config, write_random_model
    cfg = dict(COMMON, **SIZES[request.param])
    folder = write_random_model(tmp_path_factory.mktemp("layer_" + request.param), Qwen3Config(**cfg), seed=5, std=0.02,
                                norm_std=0.1)
    reqs = tiny.random_requests(cfg["vocab_size"], LENGTHS, seed=77)
    return folder, reqs, tiny.plain_logits(folder, reqs)


def test_bfloat16_cuttings_at_production_sizes(big_layer):
    from garlic_inference_b200 import AutoModel
    folder, reqs, want = big_layer
    model = AutoModel.from_pretrained(folder, device=0, dtype="bfloat16", max_tokens=2048, page_size=64)
    for what, steps in (("whole", tiny.trace_whole(reqs)), ("last 32 one by one", tiny.trace_tail_by_one(reqs, tail=32)),
                        ("unequal batches", tiny.trace_batched(reqs, [["r0", "r1", "r2"], ["r3", "r1"]], prompt_frac=0.9))):
        got = tiny.run_trace_in_process(model, steps)
        worst = tiny.compare(got, want, tiny.TOL["bfloat16"], f"production-size layer, bfloat16, {what}")
        assert worst > 1e-5, "bfloat16 cannot be this exact"
    cache = model.engine.cache
    assert cache.slots.n_free == cache.max_slots


def test_float32_at_production_sizes(big_layer):
    from garlic_inference_b200 import AutoModel
    folder, reqs, want = big_layer
    model = AutoModel.from_pretrained(folder, device=0, dtype="float32", max_tokens=1024, page_size=64)
    short = {"r1": reqs["r1"], "r3": reqs["r3"]}
    whole = tiny.run_trace_in_process(model, tiny.trace_whole(short))
    tail = tiny.run_trace_in_process(model, tiny.trace_tail_by_one(short, tail=8))
    assert tiny.compare(whole, want, tiny.TOL["float32"], "production-size layer, float32, whole") < 2e-5
    tiny.compare(tail, want, tiny.TOL["float32"], "production-size layer, float32, last 8 one by one")


@pytest.mark.parametrize("n", [20, 40, 70])
def test_batches_of_many_sequences_at_the_benchmark_s_layer_sizes(n, tmp_path_factory):
    """One layer of the benchmark model's sizes, batches of 20, 40 and 70 sequences that start together with short
    unequal prompts and decode 40 steps and more (recorded steps of 32, 64 and 128 rows), then a second batch in the
    same cache: the products that take 9 to 32 rows (the feed-forward's go to the stream-K kernel there), 33 to 64
    rows and more, at the shapes whose throughput the benchmark reports."""
    import numpy as np
    from garlic_inference_b200 import AutoModel, Qwen3Config, write_random_model
    cfg = dict(COMMON, **SIZES["8B"])
    folder = write_random_model(tmp_path_factory.mktemp("layer_8B_wide"), Qwen3Config(**cfg), seed=6, std=0.02, norm_std=0.1)
    rng = np.random.default_rng(n)
    lengths = rng.integers(48, 65, size=n + 4).tolist()
    reqs = tiny.random_requests(cfg["vocab_size"], lengths, seed=n + 1)
    ids = list(reqs)
    want = tiny.plain_logits(folder, reqs)
    model = AutoModel.from_pretrained(folder, device=0, dtype="bfloat16", max_tokens=64 * n, page_size=64)
    steps = tiny.trace_batched(reqs, [ids[:n], ids[n:]], prompt_frac=0.12)
    got = tiny.run_trace_in_process(model, steps)
    tiny.assert_covers(got, reqs)
    worst = tiny.compare(got, want, tiny.TOL["bfloat16"], f"8B-size layer, bfloat16, batch of {n}")
    print(f"8B-size layer, batch of {n}: worst relative error {worst:.3e}")
    assert max(model.engine.graphs._graphs) == 1 << (n - 1).bit_length()


def test_the_benchmark_model_s_first_two_layers_from_random(tmp_path_factory):
    """What bench.py times is `AutoModel.from_random` at Qwen3-8B sizes.  Its random weights depend on (seed, tensor
    name, index) alone, so the same model can be written to a folder and read by the plain implementation: two
    layers of it, the full vocabulary of 151,936, a prompt of 300 tokens and 8 decode steps."""
    import numpy as np
    from garlic_inference_b200 import AutoModel, Qwen3Config, write_random_model
    cfg = Qwen3Config(hidden_size=4096, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                      intermediate_size=12288, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                      max_position_embeddings=40960, tie_word_embeddings=False)
    model = AutoModel.from_random(cfg, seed=0, device=0, dtype="bfloat16", max_tokens=512)      # as bench.py makes it
    folder = write_random_model(tmp_path_factory.mktemp("bench_2_layers"), cfg, seed=0, device="cuda")
    reqs = tiny.random_requests(cfg.vocab_size, [308], seed=9)
    want = tiny.plain_logits(folder, reqs)
    steps = tiny.trace_tail_by_one(reqs, tail=8)
    got = tiny.run_trace_in_process(model, steps)
    tiny.assert_covers(got, reqs)
    worst = tiny.compare(got, want, tiny.TOL["bfloat16"], "two layers of the benchmark model, bfloat16")
    print(f"two layers of the benchmark model: worst relative error {worst:.3e}")
    assert worst > 1e-5, "bfloat16 cannot be this exact"
    top = np.stack([got["r0"][p] for p in range(308)]).argmax(1)
    margin = np.sort(want["r0"], axis=1)
    sure = (margin[:, -1] - margin[:, -2]) > 2 * tiny.TOL["bfloat16"] * np.abs(want["r0"]).max()
    assert (top[sure] == want["r0"].argmax(1)[sure]).all()
