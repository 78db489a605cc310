"""Each part of a layer alone against the plain implementation's function for it, and the generality
of the assembly: a toy mixer with state of its own (defined here, registered here, no file of the
package changed), different mixers in different layers, a layer named twice in the schedule, and a
layer that reads another layer's cache."""
import json
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import tiny

pytestmark = pytest.mark.gpu

DEV = torch.device("cuda", 0)


class DictLoader:
    """Hands a part its tensors from a dict, the way the model builder's loader does."""

    def __init__(self, tensors, rt):
        from garlic_inference_b200.weights import device_dtype
        self.t, self.rt, self._dd = tensors, rt, device_dtype

    def dtype(self, *locals_):
        kept = [self._dd(self.t[n].dtype, self.rt.dtype) for n in locals_]
        return torch.float32 if torch.float32 in kept else kept[0]

    def __call__(self, local, out=None):
        if out is not None:
            out.copy_(self.t[local])
            return out
        return self.t[local].to(device=self.rt.device, dtype=self.dtype(local)).contiguous()


def rt_for(dtype):
    from garlic_inference_b200.parts import Runtime
    return Runtime(dtype, DEV)


def rnd(shape, seed, scale=1.0, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def tol(dtype):
    return dict(rtol=3e-2, atol=3e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rms_norm_part(dtype):
    from garlic_inference_b200.parts import RMSNorm
    w = 1 + rnd((200,), 0, 0.2)
    part = RMSNorm(dict(size=200, eps=1e-4), DictLoader({"weight": w}, rt_for(dtype)), rt_for(dtype))
    res = rnd((6, 200), 1, 2.0, torch.float32).to(DEV)
    delta = rnd((6, 200), 2, 1.0, dtype).to(DEV)
    want = plain.rms_norm(res.cpu() + delta.float().cpu(), w.float(), 1e-4)
    got = part.add_norm(delta, res)
    torch.testing.assert_close(got.float().cpu(), want, **tol(dtype))


def test_rotary_part_tables():
    from garlic_inference_b200.parts import RotaryPositions
    part = RotaryPositions(dict(head_dim=48, rotary_dim=48, theta=5e5, max_positions=4000), None, rt_for(torch.float32))
    cos, sin, r = part.rotary_tables()
    ang = plain.rope_angles(torch.arange(4000), 48, 5e5, torch.float64)
    assert r == 48 and cos.shape == (4000, 24)
    torch.testing.assert_close(cos.cpu().double(), ang.cos(), rtol=0, atol=1e-7)
    torch.testing.assert_close(sin.cpu().double(), ang.sin(), rtol=0, atol=1e-7)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    from garlic_inference_b200.parts import SwiGLUMLP
    w = {"gate_proj": rnd((112, 80), 3, 0.1), "up_proj": rnd((112, 80), 4, 0.1), "down_proj": rnd((80, 112), 5, 0.1)}
    part = SwiGLUMLP(dict(hidden_size=80, intermediate_size=112), DictLoader(w, rt_for(dtype)), rt_for(dtype))
    x = rnd((13, 80), 6, 1.0, dtype)
    want = plain.swiglu_mlp(x.float(), {"p." + k + ".weight": v.float() for k, v in w.items()}, "p.")
    got = part.step(x.to(DEV), None)
    torch.testing.assert_close(got.float().cpu(), want, **tol(dtype))


def _attention_setup(dtype, window, n_q=6, n_kv=2, d=32, hidden=96, S=50, page=16):
    from garlic_inference_b200.cache import PagedCache
    from garlic_inference_b200.parts import GQAAttention, RotaryPositions, StepContext
    rt = rt_for(dtype)
    w = {"q_proj": rnd((n_q * d, hidden), 10, 0.1), "k_proj": rnd((n_kv * d, hidden), 11, 0.1),
         "v_proj": rnd((n_kv * d, hidden), 12, 0.1), "o_proj": rnd((hidden, n_q * d), 13, 0.1),
         "q_norm": 1 + rnd((d,), 14, 0.2), "k_norm": 1 + rnd((d,), 15, 0.2)}
    params = dict(hidden_size=hidden, n_heads=n_q, n_kv_heads=n_kv, head_dim=d, qk_norm=True, qk_norm_eps=1e-5,
                  window=window, softmax_scale=d ** -0.5)
    part = GQAAttention(params, DictLoader(w, rt), rt)
    rope = RotaryPositions(dict(head_dim=d, theta=1e4, max_positions=256), None, rt)
    cache = PagedCache([part.cache_requirement()], max_tokens=256, max_positions=256, dtype=dtype, device=DEV,
                       page_size=page)
    x = rnd((S, hidden), 16, 1.0, dtype)
    cfg = dict(num_attention_heads=n_q, num_key_value_heads=n_kv, head_dim=d, rms_norm_eps=1e-5, rope_theta=1e4)
    want = plain.attention_block(x.float(), {"a." + k + ".weight": v.float() for k, v in w.items()}, "a.", cfg,
                                 torch.arange(S), window)

    def ctx_for(slot, lo, hi):
        n = hi - lo
        return StepContext(n_tokens=n, tokens=torch.zeros(n, dtype=torch.int32, device=DEV),
                           tok_pos=torch.arange(lo, hi, dtype=torch.int32, device=DEV),
                           tok_slot=torch.full((n,), slot, dtype=torch.int32, device=DEV),
                           seq_slots=[slot], seq_starts=[0], seq_lens=[n], seq_past=[lo], all_single=(n == 1),
                           max_kv_len=hi, status=cache.status)
    return part, rope, cache, x.to(DEV), want, ctx_for


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 9])
def test_attention_part_whole_and_in_pieces(dtype, window):
    part, rope, cache, x, want, ctx_for = _attention_setup(dtype, window)
    S = x.shape[0]
    s = cache.alloc_slot()
    cache.prepare([s], [S])
    got = part.step(x, ctx_for(s, 0, S), cache.view(0), rope)
    cache.commit([s], [S])
    torch.testing.assert_close(got.float().cpu(), want, **tol(dtype))
    cache.free_slot(s)
    # the same in pieces of 17, 1, 1, ... from the cache
    s = cache.alloc_slot()
    outs, lo = [], 0
    for n in [17] + [1] * (S - 17):
        cache.prepare([s], [n])
        outs.append(part.step(x[lo:lo + n].contiguous(), ctx_for(s, lo, lo + n), cache.view(0), rope))
        cache.commit([s], [n])
        lo += n
    torch.testing.assert_close(torch.cat(outs).float().cpu(), want, **tol(dtype))
    cache.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_embedding_and_head_parts(dtype, model_dirs):
    """A whole pre-norm block of configuration B, then the two ends of the model, each alone."""
    from garlic_inference_b200.engine import DecoderModel
    from garlic_inference_b200.cache import PagedCache
    from garlic_inference_b200.parts import StepContext
    from garlic_inference_b200.weights import Checkpoint
    cfg_obj = tiny.make_config("B")
    d = model_dirs("B")
    cfg, w = plain.read_model_dir(d)
    model = DecoderModel(cfg_obj.plan(), Checkpoint(d), rt_for(dtype))
    ids = np.random.default_rng(5).integers(0, 1000, size=21)
    S = len(ids)
    cache = PagedCache(model.cache_requirements(), max_tokens=64, max_positions=256, dtype=dtype, device=DEV, page_size=16)
    s = cache.alloc_slot()
    cache.prepare([s], [S])
    ctx = StepContext(n_tokens=S, tokens=torch.tensor(ids, dtype=torch.int32, device=DEV),
                      tok_pos=torch.arange(S, dtype=torch.int32, device=DEV),
                      tok_slot=torch.full((S,), s, dtype=torch.int32, device=DEV), seq_slots=[s], seq_starts=[0],
                      seq_lens=[S], seq_past=[0], max_kv_len=S, status=cache.status)
    residual = model.embedding.step(ctx)
    h0 = plain.embed(torch.tensor(ids), w["model.embed_tokens.weight"])
    assert torch.equal(residual.cpu(), h0)
    delta = model.blocks[1].step(None, residual, ctx, cache.view(1), True)
    h1 = plain.decoder_layer(h0, w, 1, cfg, torch.arange(S))
    torch.testing.assert_close(residual.cpu() + delta.float().cpu(), h1, **tol(dtype))
    rows = torch.tensor([S - 1, 0], dtype=torch.int32, device=DEV)
    normed = model.final_norm.add_norm(delta, residual, rows=rows)
    logits = model.head.step(normed)
    want = plain.output_head(h1[[S - 1, 0]], w, cfg)
    assert logits.dtype == torch.float32
    torch.testing.assert_close(logits.cpu(), want, **tol(dtype))
    cache.check_status()


# ---------------------------------------------------------------------------------------------------
# generality: a toy mixer with state, registered from outside; layer order as data
# ---------------------------------------------------------------------------------------------------
def _toy_classes():
    """A mixer whose only memory is a running sum of its inputs per sequence, kept in the cache's
    fixed-size state region, and a configuration that alternates it with attention."""
    from garlic_inference_b200 import Qwen3Config, register_architecture, register_part
    from garlic_inference_b200.cache import StateRequirement
    from garlic_inference_b200.config import ScheduleEntry
    from garlic_inference_b200.config.base import PartSpec
    from garlic_inference_b200.parts import Mixer
    from garlic_inference_b200.weights import TensorWant
    import dataclasses

    class RunningSumMixer(Mixer):
        kind = "toy_running_sum"
        graph_safe = True              # a step of one token per sequence runs from the device tensors alone

        @classmethod
        def wanted(cls, params):
            return {"mix": TensorWant((params["hidden_size"],), "norm")}

        def __init__(self, params, load, rt):
            super().__init__(params, load, rt)
            self.hidden = params["hidden_size"]
            self.decay = params["decay"]
            self.mix = load("mix").float()

        def cache_requirement(self):
            return StateRequirement((self.hidden,), torch.float32)

        def step(self, x, ctx, cache, position, writes_cache=True):
            if ctx.all_single:
                # one row per sequence, maybe recorded into a CUDA graph: row i belongs to slot tok_slot[i]; a
                # padding row's slot is -1, the state region's spare last row
                slots = ctx.tok_slot.long()
                state = cache.state[slots] * self.decay + x.float()
                cache.state[slots] = state
                return (state * self.mix).to(x.dtype)
            out = torch.empty_like(x)
            for slot, start, n in zip(ctx.seq_slots, ctx.seq_starts, ctx.seq_lens):
                state = cache.state[slot]
                for t in range(start, start + n):                 # tokens of a sequence in order
                    state = state * self.decay + x[t].float()
                    out[t] = (state * self.mix).to(x.dtype)
                cache.state[slot] = state
            return out

    class ToyConfig(Qwen3Config):
        def plan(self):
            base = super().plan()
            layers = list(base.layers)
            for i in range(1, len(layers), 2):
                toy = PartSpec("toy_running_sum", dict(hidden_size=self.hidden_size, decay=0.9),
                               dict(mix=f"model.layers.{i}.toy.mix"))
                layers[i] = dataclasses.replace(layers[i], mixer=toy, position=None)
            return dataclasses.replace(base, architecture="ToyStateForCausalLM", layers=tuple(layers))

    register_part("toy_running_sum", RunningSumMixer)
    register_architecture("ToyStateForCausalLM", ToyConfig)
    return ToyConfig


def _plain_toy_forward(cfg, w, ids):
    ids = torch.as_tensor(ids)
    pos = torch.arange(len(ids))
    h = plain.embed(ids, w["model.embed_tokens.weight"])
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        if i % 2 == 0:
            h = plain.decoder_layer(h, w, i, cfg, pos)
            continue
        x = plain.rms_norm(h, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        state, mixed = torch.zeros(cfg["hidden_size"]), []
        for t in range(len(ids)):
            state = state * 0.9 + x[t]
            mixed.append(state * w[p + "toy.mix"])
        r = torch.stack(mixed) + h
        x = plain.rms_norm(r, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        h = plain.swiglu_mlp(x, w, p + "mlp.") + r
    return plain.output_head(h, w, cfg)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_mixer_with_state_is_registered_built_and_stepped(dtype, tmp_path):
    from garlic_inference_b200 import AutoModel, write_random_model
    ToyConfig = _toy_classes()
    cfg_obj = ToyConfig(**{**tiny.TINY["B"]["cfg"], "num_hidden_layers": 4, "architectures": ["ToyStateForCausalLM"]})
    d = write_random_model(tmp_path / "toy", cfg_obj, seed=3, std=0.05, norm_std=0.2)
    assert json.loads((d / "config.json").read_text())["architectures"] == ["ToyStateForCausalLM"]
    model = AutoModel.from_pretrained(d, device=0, dtype=dtype, max_tokens=512, page_size=16)
    assert type(model.config) is ToyConfig
    cache = model.engine.cache
    assert cache.state_bytes_per_slot == 2 * 96 * 4 and len(cache.groups) == 1 and len(cache.groups[0].entries) == 2
    cfg, w = plain.read_model_dir(d)
    reqs = tiny.random_requests(1000, [40, 9, 70, 33], seed=21)
    want = {rid: _plain_toy_forward(cfg, w, t).numpy() for rid, t in reqs.items()}
    for steps in (tiny.trace_whole(reqs), tiny.trace_tail_by_one(reqs, tail=32),
                  tiny.trace_batched(reqs, [["r0", "r1"], ["r2", "r3"]])):       # slots, and their state, used again
        got = tiny.run_trace_in_process(model, steps)
        tiny.assert_covers(got, reqs)
        tiny.compare(got, want, tiny.TOL[dtype], f"toy {dtype}")
    # one layer with state of its own does not send the model back to launch-by-launch decoding
    assert model.engine.graphs is not None and sorted(model.engine.graphs._graphs) == [1, 2]


def _plain_layer(h, w, i, cfg, pos, kv=None):
    """plain.decoder_layer with the keys and values handed in (a reader of another layer's cache)
    or handed out."""
    p = f"model.layers.{i}."
    a = p + "self_attn."
    n_q, n_kv, d, eps, theta = (cfg[k] for k in ("num_attention_heads", "num_key_value_heads", "head_dim",
                                                 "rms_norm_eps", "rope_theta"))
    S = h.shape[0]
    x = plain.rms_norm(h, w[p + "input_layernorm.weight"], eps)
    q = plain.apply_rope(plain.rms_norm((x @ w[a + "q_proj.weight"].T).view(S, n_q, d), w[a + "q_norm.weight"], eps), pos, theta)
    if kv is None:
        k = plain.apply_rope(plain.rms_norm((x @ w[a + "k_proj.weight"].T).view(S, n_kv, d), w[a + "k_norm.weight"], eps), pos, theta)
        v = (x @ w[a + "v_proj.weight"].T).view(S, n_kv, d)
        kv = (k, v)
    o = plain.attention_scores(q, kv[0], kv[1]).reshape(S, n_q * d) @ w[a + "o_proj.weight"].T
    r = o + h
    x = plain.rms_norm(r, w[p + "post_attention_layernorm.weight"], eps)
    return plain.swiglu_mlp(x, w, p + "mlp.") + r, kv


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_order_is_data(dtype, tmp_path):
    """Schedule: layer 0, layer 1, layer 0 again (its weights shared, a cache entry of its own), then
    layer 2 reading the cache that layer 1 wrote."""
    import dataclasses
    from garlic_inference_b200 import AutoModel, Qwen3Config, register_architecture, write_random_model
    from garlic_inference_b200.config import ScheduleEntry

    class LoopedConfig(Qwen3Config):
        def plan(self):
            base = super().plan()
            sched = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2), ScheduleEntry(2, 1, writes_cache=False))
            return dataclasses.replace(base, schedule=sched)

    register_architecture("LoopedForCausalLM", LoopedConfig)
    cfg_obj = LoopedConfig(**{**tiny.TINY["A"]["cfg"], "num_hidden_layers": 3, "architectures": ["LoopedForCausalLM"]})
    d = write_random_model(tmp_path / "looped", cfg_obj, seed=4, std=0.05, norm_std=0.2)
    model = AutoModel.from_pretrained(d, device=0, dtype=dtype, max_tokens=512, page_size=16)
    assert len(model.engine.cache.groups[0].entries) == 3
    cfg, w = plain.read_model_dir(d)

    def plain_forward(ids):
        ids = torch.as_tensor(ids)
        pos = torch.arange(len(ids))
        h = plain.embed(ids, w["model.embed_tokens.weight"])
        h, _ = _plain_layer(h, w, 0, cfg, pos)
        h, kv1 = _plain_layer(h, w, 1, cfg, pos)
        h, _ = _plain_layer(h, w, 0, cfg, pos)
        h, _ = _plain_layer(h, w, 2, cfg, pos, kv=kv1)
        return plain.output_head(h, w, cfg)

    reqs = tiny.random_requests(512, [50, 7, 90], seed=22)
    want = {rid: plain_forward(t).numpy() for rid, t in reqs.items()}
    for steps in (tiny.trace_whole(reqs), tiny.trace_tail_by_one(reqs, tail=32),
                  tiny.trace_batched(reqs, [["r0", "r1", "r2"]])):
        got = tiny.run_trace_in_process(model, steps)
        tiny.assert_covers(got, reqs)
        tiny.compare(got, want, tiny.TOL[dtype], f"looped {dtype}")


# ---------------------------------------------------------------------------------------------------
# generality: a toy feed-forward with routing and a toy position encoding, registered from outside
# ---------------------------------------------------------------------------------------------------
def _toy_routed_classes():
    """A feed-forward that sends every token to one of three small experts (the router's largest logit, ties to
    the lowest index, router in float32), and learned absolute positions added to the embedded tokens in place
    of rotations.  Both live in this test; the framework's files do not know them."""
    import dataclasses
    from garlic_inference_b200 import Qwen3Config, register_architecture, register_part
    from garlic_inference_b200.config.base import PartSpec
    from garlic_inference_b200.parts import FeedForward, PositionEncoding
    from garlic_inference_b200.weights import TensorWant

    class Top1Experts(FeedForward):
        kind = "toy_top1_experts"

        @classmethod
        def wanted(cls, params):
            h, e, w = params["hidden_size"], params["n_experts"], params["expert_width"]
            return {"router": TensorWant((e, h)), "w_in": TensorWant((e * w, h)), "w_out": TensorWant((e * h, w))}

        def __init__(self, params, load, rt):
            super().__init__(params, load, rt)
            self.h, self.e, self.w = params["hidden_size"], params["n_experts"], params["expert_width"]
            self.router = load("router").float()
            self.w_in = load("w_in").float().view(self.e, self.w, self.h)
            self.w_out = load("w_out").float().view(self.e, self.h, self.w)

        def step(self, x, ctx):
            xf = x.float()
            choice = (xf @ self.router.T).argmax(dim=-1)          # first maximum = lowest index
            out = torch.zeros_like(xf)
            for e in range(self.e):                               # tokens gathered per expert, results scattered back
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    hid = torch.relu(xf[rows] @ self.w_in[e].T)
                    out[rows] = hid @ self.w_out[e].T
            return out.to(x.dtype)

    class LearnedPositions(PositionEncoding):
        kind = "toy_learned_positions"

        @classmethod
        def wanted(cls, params):
            return {"table": TensorWant((params["max_positions"], params["hidden_size"]))}

        def __init__(self, params, load, rt):
            super().__init__(params, load, rt)
            self.table = load("table").float()

        def on_embedding(self, residual, ctx):
            residual += self.table[ctx.tok_pos.long()]            # padding rows get position 0: they are nobody's rows

    class RoutedConfig(Qwen3Config):
        def plan(self):
            base = super().plan()
            layers = []
            for i, layer in enumerate(base.layers):
                ff = PartSpec("toy_top1_experts", dict(hidden_size=self.hidden_size, n_experts=3, expert_width=40),
                              {k: f"model.layers.{i}.experts.{k}" for k in ("router", "w_in", "w_out")})
                layers.append(dataclasses.replace(layer, feed_forward=ff if i % 2 == 0 else layer.feed_forward,
                                                  position="learned"))
            positions = {"learned": PartSpec("toy_learned_positions",
                                             dict(max_positions=self.max_position_embeddings, hidden_size=self.hidden_size),
                                             dict(table="model.positions.weight"))}
            return dataclasses.replace(base, architecture="ToyRoutedForCausalLM", layers=tuple(layers), positions=positions)

    register_part("toy_top1_experts", Top1Experts)
    register_part("toy_learned_positions", LearnedPositions)
    register_architecture("ToyRoutedForCausalLM", RoutedConfig)
    return RoutedConfig


def _plain_routed_forward(cfg, w, ids):
    """The same model, plainly: learned positions on the embedding, attention without rotation, experts on the
    even layers."""
    ids = torch.as_tensor(ids)
    n = len(ids)
    h = plain.embed(ids, w["model.embed_tokens.weight"]) + w["model.positions.weight"][:n].float()
    d, n_q, n_kv = cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        x = plain.rms_norm(h, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        q = (x @ w[p + "self_attn.q_proj.weight"].float().T).view(n, n_q, d)
        k = (x @ w[p + "self_attn.k_proj.weight"].float().T).view(n, n_kv, d)
        v = (x @ w[p + "self_attn.v_proj.weight"].float().T).view(n, n_kv, d)
        q = plain.rms_norm(q, w[p + "self_attn.q_norm.weight"], cfg["rms_norm_eps"])
        k = plain.rms_norm(k, w[p + "self_attn.k_norm.weight"], cfg["rms_norm_eps"])
        o = plain.attention_scores(q, k, v, None)
        r = o.reshape(n, n_q * d) @ w[p + "self_attn.o_proj.weight"].float().T + h
        x = plain.rms_norm(r, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        if i % 2 == 0:
            router = w[p + "experts.router"].float()
            w_in = w[p + "experts.w_in"].float().view(3, 40, -1)
            w_out = w[p + "experts.w_out"].float().view(3, -1, 40)
            choice = (x @ router.T).argmax(dim=-1)
            m = torch.stack([torch.relu(x[t] @ w_in[c].T) @ w_out[c].T for t, c in enumerate(choice.tolist())])
        else:
            m = plain.swiglu_mlp(x, w, p + "mlp.")
        h = m + r
    return plain.output_head(h, w, cfg)


def test_a_toy_routed_feed_forward_and_learned_positions_are_registered_built_and_stepped(tmp_path):
    from garlic_inference_b200 import AutoModel, write_random_model
    RoutedConfig = _toy_routed_classes()
    cfg_obj = RoutedConfig(**{**tiny.TINY["A"]["cfg"], "num_hidden_layers": 3, "max_position_embeddings": 96,
                              "architectures": ["ToyRoutedForCausalLM"]})
    d = write_random_model(tmp_path / "routed", cfg_obj, seed=8, std=0.08, norm_std=0.1)
    model = AutoModel.from_pretrained(d, device=0, dtype="float32", max_tokens=512, page_size=16)
    assert type(model.config) is RoutedConfig
    cfg, w = plain.read_model_dir(d)
    assert "model.layers.0.experts.router" in w and "model.layers.1.experts.router" not in w
    assert "model.layers.0.mlp.gate_proj.weight" not in w, "a layer's feed-forward weights are those of its own part"
    reqs = tiny.random_requests(512, [30, 7, 64, 21], seed=31)
    want = {rid: _plain_routed_forward(cfg, w, t).numpy() for rid, t in reqs.items()}
    for steps in (tiny.trace_whole(reqs), tiny.trace_tail_by_one(reqs, tail=16),
                  tiny.trace_batched(reqs, [["r0", "r1"], ["r2", "r3"]])):
        got = tiny.run_trace_in_process(model, steps)
        tiny.assert_covers(got, reqs)
        tiny.compare(got, want, tiny.TOL["float32"], "toy routed float32")


# ---------------------------------------------------------------------------------------------------
# generality: a toy norm, a toy block arrangement and a partial rotation, registered from outside
# ---------------------------------------------------------------------------------------------------
def _toy_parallel_classes():
    """The two remaining kinds of part, defined here: a norm that subtracts the mean and has a bias, and a block
    that runs its mixer and its feed-forward side by side on one normed input (h += attention(x) + ffn(x)); and the
    built-in rotary part asked to rotate only the first half of every head.  The framework's files know none of it."""
    import dataclasses
    from garlic_inference_b200 import Qwen3Config, register_architecture, register_part
    from garlic_inference_b200.config.base import LayerSpec, PartSpec
    from garlic_inference_b200.parts import Block, Norm
    from garlic_inference_b200.weights import TensorWant

    class MeanNorm(Norm):
        kind = "toy_mean_norm"
        graph_safe = True                   # device tensors only

        @classmethod
        def wanted(cls, params):
            return {"weight": TensorWant((params["size"],), "norm"), "bias": TensorWant((params["size"],))}

        def __init__(self, params, load, rt):
            super().__init__(params, load, rt)
            self.eps = params["eps"]
            self.weight, self.bias = load("weight").float(), load("bias").float()

        def add_norm(self, delta, residual, rows=None, write_residual=True):
            s = residual if rows is None else residual.index_select(0, rows.long())
            if delta is not None:
                s = s + (delta if rows is None else delta.index_select(0, rows.long())).float()
                if write_residual and rows is None:
                    residual.copy_(s)
            mu = s.mean(-1, keepdim=True)
            var = ((s - mu) ** 2).mean(-1, keepdim=True)
            return ((s - mu) * torch.rsqrt(var + self.eps) * self.weight + self.bias).to(self.rt.dtype)

    class ParallelBlock(Block):
        kind = "toy_parallel"

        def __init__(self, mixer, feed_forward, norms, position, rt):
            self.rt, self.mixer, self.feed_forward, self.position = rt, mixer, feed_forward, position
            self.norm = norms["input"]

        @property
        def graph_safe(self):
            return all(p.graph_safe for p in (self.mixer, self.feed_forward, self.norm, self.position))

        def cache_requirement(self):
            return self.mixer.cache_requirement()

        def step_arrays(self, shape, cache):
            return {**self.mixer.step_arrays(shape, cache), **self.feed_forward.step_arrays(shape, cache)}

        def step(self, delta, residual, ctx, cache, writes_cache=True):
            x = self.norm.add_norm(delta, residual)
            return self.mixer.step(x, ctx, cache, self.position, writes_cache) + self.feed_forward.step(x, ctx)

    class ParallelConfig(Qwen3Config):
        def plan(self):
            base = super().plan()
            ln = lambda prefix: PartSpec("toy_mean_norm", dict(size=self.hidden_size, eps=self.rms_norm_eps),
                                         dict(weight=prefix + ".weight", bias=prefix + ".bias"))
            layers = tuple(LayerSpec("toy_parallel", l.mixer, l.feed_forward,
                                     {"input": ln(f"model.layers.{i}.input_layernorm")}, position="rotary")
                           for i, l in enumerate(base.layers))
            positions = {"rotary": dataclasses.replace(
                base.positions["rotary"], params={**base.positions["rotary"].params, "rotary_dim": self.head_dim // 2})}
            return dataclasses.replace(base, architecture="ToyParallelForCausalLM", layers=layers, positions=positions,
                                       final_norm=ln("model.norm"))

    register_part("toy_mean_norm", MeanNorm)
    register_part("toy_parallel", ParallelBlock)
    register_architecture("ToyParallelForCausalLM", ParallelConfig)
    return ParallelConfig


def _plain_parallel_forward(cfg, w, ids):
    ids = torch.as_tensor(ids)
    n = len(ids)
    pos = torch.arange(n)
    d, n_q, n_kv, eps, theta = (cfg[k] for k in ("head_dim", "num_attention_heads", "num_key_value_heads",
                                                 "rms_norm_eps", "rope_theta"))

    def mean_norm(x, prefix):
        mu = x.mean(-1, keepdim=True)
        var = ((x - mu) ** 2).mean(-1, keepdim=True)
        return (x - mu) * torch.rsqrt(var + eps) * w[prefix + ".weight"] + w[prefix + ".bias"]

    def half_rope(x):                        # the first d/2 of every head rotated (angles theta^(-2i/(d/2))), the rest as it is
        return torch.cat([plain.apply_rope(x[..., : d // 2], pos, theta), x[..., d // 2:]], dim=-1)

    h = plain.embed(ids, w["model.embed_tokens.weight"])
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        x = mean_norm(h, p + "input_layernorm")
        q = plain.rms_norm((x @ w[p + "self_attn.q_proj.weight"].T).view(n, n_q, d), w[p + "self_attn.q_norm.weight"], eps)
        k = plain.rms_norm((x @ w[p + "self_attn.k_proj.weight"].T).view(n, n_kv, d), w[p + "self_attn.k_norm.weight"], eps)
        v = (x @ w[p + "self_attn.v_proj.weight"].T).view(n, n_kv, d)
        a = plain.attention_scores(half_rope(q), half_rope(k), v).reshape(n, n_q * d) @ w[p + "self_attn.o_proj.weight"].T
        h = h + a + plain.swiglu_mlp(x, w, p + "mlp.")
    return mean_norm(h, "model.norm") @ w["lm_head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_norm_a_toy_block_and_a_partial_rotation(dtype, tmp_path):
    from garlic_inference_b200 import AutoModel, write_random_model
    ParallelConfig = _toy_parallel_classes()
    cfg_obj = ParallelConfig(**{**tiny.TINY["B"]["cfg"], "num_hidden_layers": 2, "architectures": ["ToyParallelForCausalLM"]})
    d = write_random_model(tmp_path / "parallel", cfg_obj, seed=12, std=0.05, norm_std=0.2)
    model = AutoModel.from_pretrained(d, device=0, dtype=dtype, max_tokens=512, page_size=16)
    assert type(model.config) is ParallelConfig
    cfg, w = plain.read_model_dir(d)
    assert "model.layers.1.input_layernorm.bias" in w and "model.layers.1.post_attention_layernorm.weight" not in w
    reqs = tiny.random_requests(1000, [45, 8, 70, 33], seed=51)
    want = {rid: _plain_parallel_forward(cfg, w, t).numpy() for rid, t in reqs.items()}
    for steps in (tiny.trace_whole(reqs), tiny.trace_tail_by_one(reqs, tail=32),
                  tiny.trace_batched(reqs, [["r0", "r1"], ["r2", "r3"]])):
        got = tiny.run_trace_in_process(model, steps)
        tiny.assert_covers(got, reqs)
        tiny.compare(got, want, tiny.TOL[dtype], f"toy parallel {dtype}")
    assert model.engine.graphs is not None and model.engine.graphs._graphs, "its decode steps were recorded"
