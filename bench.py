#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3-8B layer sizes with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

One JSON line on stdout.  `value` is decoded tokens a second at batch 8 with 2,048 cached tokens
per sequence (a step = one decode step of the whole batch), timed on the device with the sampler's
tokens fed back on the device; `e2e` is the same through `LanguageModel.generate` (prompts and
generated ids on the host, every step's ids read back), over the last K of W + K + 1 steps.  The
defaults are 128 steps after 32 warm-up steps: the first twenty or so decode steps right after the prompt
passes take 4.1 to 4.4 ms instead of 3.8 (measured; they do not when the GPU rests half a second in
between, so it is the state the power cap leaves the GPU in, not the engine).  `prefill` is one 2,048-token prompt, `points` decoding at batch 1 and 64, `roofline` the bytes a
decode step has to read (every weight once, the cache of the live requests) over its time against the measured copy bandwidth.

The library runs on one GPU: for --gpus > 1 a line says so and the exit code is 2.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# layer sizes of the benchmark configuration (Qwen3-8B): 36 layers of hidden 4096, 32 query and 8
# key/value heads of 128, feed-forward 12288, vocabulary 151936, separate head
QWEN3_8B = dict(hidden_size=4096, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
                head_dim=128, intermediate_size=12288, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                max_position_embeddings=40960, tie_word_embeddings=False)
CONTEXT = 4096          # tokens per sequence the benchmark's context allows
CACHED = 2048           # tokens each sequence holds when decoding is timed
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            p = json.load(open(path))
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                    "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained") or 0) or None, "source": "measured"}
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi in the background while a region is timed (reads only; nothing is set).  Every sample carries
    nvidia-smi's own wall-clock time, so that a summary can be taken over a part of the sampled time."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw")

    def __init__(self, gpu_id: str, period_ms: int = 100):
        self.gpu_id, self.period_ms, self.proc, self.lines = gpu_id, period_ms, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.gpu_id, f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        self.lines += [l for l in out.splitlines() if l.strip()]
        self.proc = None

    def summary(self, since: float = None, until: float = None):
        """Median SM clock and the reasons seen, over all samples or over those taken between two time.time() values."""
        import datetime
        sm, mx, watts, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            try:
                if since is not None or until is not None:
                    t = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    if (since is not None and t < since) or (until is not None and t > until):
                        continue
                sm.append(float(f[1])), mx.append(float(f[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, f[3:7]):
                if v.lower() == "active":
                    reasons.add(name)
            try:
                watts.append(float(f[7]))
            except (ValueError, IndexError):
                pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
        if watts:
            out["watts"] = statistics.median(watts)
        return out


def decode_step_bytes(cfg, n_layers, batch, context_tokens):
    """Bytes one decode step has to read: every weight it uses once (bfloat16), the embedding rows of the
    batch, and the keys and values of the live requests."""
    h, d = cfg["hidden_size"], cfg["head_dim"]
    n_q, n_kv, inter, vocab = (cfg[k] for k in ("num_attention_heads", "num_key_value_heads", "intermediate_size",
                                                "vocab_size"))
    per_layer = ((n_q + 2 * n_kv) * d * h + h * n_q * d + 3 * inter * h + 2 * h + 2 * d) * 2
    weights = n_layers * per_layer + (vocab * h + h) * 2 + batch * h * 2
    kv = batch * context_tokens * n_layers * 2 * n_kv * d * 2
    return weights + kv, weights, kv


def prefill_flops(cfg, n_layers, tokens):
    h, d = cfg["hidden_size"], cfg["head_dim"]
    n_q, n_kv, inter, vocab = (cfg[k] for k in ("num_attention_heads", "num_key_value_heads", "intermediate_size",
                                                "vocab_size"))
    linear = 2 * tokens * ((n_q + 2 * n_kv) * d * h + h * n_q * d + 3 * inter * h)
    attn = 4 * n_q * d * tokens * (tokens + 1) // 2
    return n_layers * (linear + attn) + 2 * vocab * h


REFERENCE_RUNNER = os.path.join(ROOT, "baseline", "_ref", "bin", "reference_runner")


def write_reference_model(folder, n_layers):
    """An 8B-size folder for upstream's loader: the same tensors and shapes as the benchmark model, values
    N(0, 0.02) drawn by torch on the GPU, norm weights 1, and `tie_word_embeddings` true because upstream
    always uses the embedding table as the head (src/models/qwen3/qwen3.cpp:58): a decode step reads the same
    bytes.  Nothing of this repository's compiled library is used."""
    import torch
    from garlic_inference_b200 import Qwen3Config
    from garlic_inference_b200.engine.model import wanted_tensors
    from garlic_inference_b200.weights.safetensors_io import write_safetensors_lazy
    cfg = Qwen3Config(**{**QWEN3_8B, "num_hidden_layers": n_layers, "tie_word_embeddings": True})
    wants = wanted_tensors(cfg.plan())
    gen = torch.Generator(device="cuda").manual_seed(0)

    def make(name):
        w = wants[name]
        if w.role == "norm":
            return torch.ones(tuple(w.shape), dtype=torch.bfloat16)
        t = torch.randn(tuple(w.shape), generator=gen, device="cuda", dtype=torch.bfloat16).mul_(0.02)
        return t.cpu()

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    write_safetensors_lazy(os.path.join(folder, "model.safetensors"),
                           {n: (torch.bfloat16, tuple(w.shape)) for n, w in wants.items()}, make)
    torch.cuda.empty_cache()


def reference_arm(args) -> int:
    """Upstream's own dense Qwen3 code (built unmodified for sm_100a by baseline/build_reference.py, with the
    driver baseline/reference_driver.cpp) on the benchmark's workload: the same JSON line, `impl: reference`."""
    import shutil
    import tempfile

    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    if not os.path.isfile(REFERENCE_RUNNER):
        src = os.environ.get("GARLIC_REFERENCE_SRC", os.path.join(os.path.dirname(ROOT), "reference"))
        if not os.path.isdir(src):
            return unavailable("baseline/_ref/bin/reference_runner is not built and there is no upstream checkout "
                               "here to build it from (baseline/build_reference.py)")
        r = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "build_reference.py"), "--src", src],
                           capture_output=True, text=True)
        if r.returncode != 0 or not os.path.isfile(REFERENCE_RUNNER):
            return unavailable("building upstream's dense path failed: " + (r.stderr or r.stdout).strip()[-300:].replace("\n", " "))
    import torch
    if not torch.cuda.is_available():
        return unavailable("no GPU here")
    K, W = args.steps, max(args.warmup, 3)
    n_layers = args.layers or QWEN3_8B["num_hidden_layers"]
    pk = peaks()
    props = torch.cuda.get_device_properties(0)
    gpu_id = "GPU-" + str(props.uuid) if getattr(props, "uuid", None) else "0"
    need = 2.2 * (n_layers * 385.9e6 + 1.25e9)                  # the file, with room to spare
    base = next((d for d in ("/dev/shm", tempfile.gettempdir()) if os.path.isdir(d) and shutil.disk_usage(d).free > need), None)
    if base is None:
        return unavailable("no temporary folder with %.0f GB free for the model file" % (need / 1e9))
    folder = tempfile.mkdtemp(prefix="garlic_ref_model_", dir=base)
    try:
        t0 = time.time()
        write_reference_model(folder, n_layers)
        print(f"bench.py: wrote the model folder in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)

        def run(batch, chunk, steps, warmup, repeats=0, clocks=None):
            cmd = [REFERENCE_RUNNER, folder, "--batch", str(batch), "--prompt-len", str(CACHED), "--chunk", str(chunk),
                   "--steps", str(steps), "--warmup", str(warmup), "--prefill-repeats", str(repeats)]
            if clocks:
                clocks.start()
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=1200)
            if clocks:
                clocks.stop()
            if r.returncode != 0:
                raise RuntimeError(f"reference_runner exited with {r.returncode}: {(r.stderr or r.stdout).strip()[-300:]}")
            return json.loads(r.stdout.strip().splitlines()[-1])

        clocks = ClockSampler(gpu_id)
        try:
            main_run = run(args.batch, 1024 if args.batch * CACHED * QWEN3_8B["vocab_size"] >= 2 ** 31 else CACHED, K, W,
                           clocks=clocks)
            pre = run(1, PREFILL_TOKENS, 0, 0, repeats=4)
            points = {}
            for b, chunk in (() if args.no_points else ((1, CACHED), (64, 128))):
                try:                                   # a point that cannot run (memory) leaves the others standing
                    points[f"decode_b{b}"] = b * 1e3 / run(b, chunk, K, W)["decode_ms_per_step"]
                except RuntimeError as e:
                    points[f"decode_b{b}_unavailable"] = str(e)[:200]
        except (RuntimeError, subprocess.TimeoutExpired, ValueError, IndexError) as e:
            return unavailable(str(e).replace("\n", " ")[:400])
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    ms = main_run["decode_ms_per_step"]
    pre_ms = statistics.median(pre["prefill_ms"][1:])
    total_b, weight_b, _ = decode_step_bytes(QWEN3_8B, n_layers, args.batch, CACHED + W + (K + 1) / 2)
    achieved = total_b / (ms / 1e3) / 1e9
    line = {
        "impl": "reference",
        "metric": f"decode tok/s at batch {args.batch} (Qwen3-8B layer sizes, {CACHED} cached tokens per sequence)",
        "value": args.batch * 1e3 / ms, "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02) in a model folder, token ids from a counter; the head is tied "
                "because upstream always ties it (the same bytes are read per step)",
        "config": {"model": "Qwen3-8B layer sizes", "global_batch": args.batch, "seq_len": CONTEXT,
                   "cached_tokens": CACHED, "parallelism": "none (1 GPU)", "layers_run": n_layers,
                   "layers_config": QWEN3_8B["num_hidden_layers"], "hidden_size": 4096, "n_heads": 32,
                   "n_kv_heads": 8, "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936,
                   "page_size": 32, "sampling": "upstream's argmax, result read by the host every step",
                   "prompt_chunk": main_run["chunk"],
                   "l2": "inputs exceed L2: a step reads %.1f GB of weights" % (weight_b / 1e9)},
        "clocks": clocks.summary(),
        # upstream's loop is synchronous: every step copies positions and block tables to the device and reads the
        # argmax back, so the wall clock over the same steps is its end-to-end figure
        "e2e": {"value": args.batch * 1e3 / main_run["decode_wall_ms_per_step"], "unit": "tokens/s",
                "h2d_bytes_per_step": main_run["h2d_bytes_per_step"], "d2h_bytes_per_step": main_run["d2h_bytes_per_step"]},
        "gpu_launches": 0,
        "prefill": {"value": PREFILL_TOKENS / (pre_ms / 1e3), "tokens": PREFILL_TOKENS, "ms": pre_ms,
                    "frac": (prefill_flops(QWEN3_8B, n_layers, PREFILL_TOKENS) + 2 * (PREFILL_TOKENS - 1) * 151936 * 4096)
                    / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12),
                    "note": "upstream computes logits at all 2,048 positions and reads 2,048 argmax results back"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "bytes_per_step": total_b, "peaks": pk["source"]},
        "points": points,
        "memory": {"free_gb_after_prompt": main_run["free_gb_after_prompt"], "free_gb_at_end": main_run["free_gb_at_end"]},
    }
    print(json.dumps(line))
    return 0


# the two larger workloads (layer sizes of Qwen3-14B and Qwen3-32B), run through `generate()`
LARGER = {
    "qwen3_14b": dict(cfg=dict(hidden_size=5120, num_hidden_layers=40, num_attention_heads=40, num_key_value_heads=8,
                               head_dim=128, intermediate_size=17408, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                               max_position_embeddings=40960, tie_word_embeddings=False),
                      batch=16, prompt=(256, 2048), new_tokens=512),
    "qwen3_32b": dict(cfg=dict(hidden_size=5120, num_hidden_layers=64, num_attention_heads=64, num_key_value_heads=8,
                               head_dim=128, intermediate_size=25600, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                               max_position_embeddings=40960, tie_word_embeddings=False),
                      batch=32, prompt=(1024, 1024), new_tokens=1024),
}


def larger_workloads(first_model, pk, gpu_id) -> dict:
    """Batch 16 with prompts uniform in [256, 2,048] then 512 decode steps at Qwen3-14B layer sizes; batch 32 with
    prompts of 1,024 then 1,024 decode steps at Qwen3-32B layer sizes (65.5 GB of weights).  Random weights, all
    layers, through `LanguageModel.generate` (host ids in and out).  Decode figures are over all decode steps."""
    import gc
    import torch
    from garlic_inference_b200 import LanguageModel, Qwen3Config
    # the benchmark model leaves the device before the larger ones arrive
    first_model.engine.graphs = None
    first_model.engine.cache = None
    first_model.engine.model = None
    first_model.model = None
    gc.collect()
    torch.cuda.empty_cache()
    out = {}
    gen = torch.Generator().manual_seed(1)
    for name, w in LARGER.items():
        cfg = Qwen3Config(**w["cfg"])
        lo, hi = w["prompt"]
        lens = [lo] * w["batch"] if lo == hi else torch.randint(lo, hi + 1, (w["batch"],), generator=gen).tolist()
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist() for n in lens]
        per_seq = [-(-(n + w["new_tokens"]) // 64) * 64 for n in lens]
        try:
            model = LanguageModel.from_random(cfg, seed=0, device=0, dtype="bfloat16", max_tokens=sum(per_seq) + 64)
            model.generate([p[:64] for p in prompts], max_new_tokens=8)             # records the decode step, warms the path
            clocks = ClockSampler(gpu_id, period_ms=50)
            clocks.start()
            toks = model.generate(prompts, max_new_tokens=w["new_tokens"])
            clocks.stop()
            st = model.last_stats
            assert all(len(t) == w["new_tokens"] for t in toks)
            steps = len(st.step_times) - 1                                          # decode steps (the first time is the prompt step's)
            seconds = st.step_times[-1] - st.step_times[0]
            ctx = sum(lens) / len(lens) + steps / 2
            total_b, weight_b, kv_b = decode_step_bytes(w["cfg"], cfg.num_hidden_layers, w["batch"], ctx)
            ms = 1e3 * seconds / steps
            out[name] = {"batch": w["batch"], "prompt_tokens": sum(lens), "decode_steps": steps, "layers": cfg.num_hidden_layers,
                         "decode_tok_s": w["batch"] * steps / seconds, "ms_per_step": ms,
                         "prefill_tok_s": sum(lens) / st.prefill_seconds if st.prefill_seconds else None,
                         "bytes_per_step": total_b, "hbm_frac": total_b / (ms / 1e3) / 1e9 / pk["hbm_gbs"],
                         "weights_gb": weight_b / 1e9, "sm_mhz": clocks.summary().get("sm_mhz")}
            model.engine.check()
        except Exception as e:                                                      # a point that cannot run leaves the line standing
            out[name] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        model = None
        gc.collect()
        torch.cuda.empty_cache()
    return out


def study_prefill_clocks(model, prompt, gpu_id, flops) -> int:
    """How a prompt step's time follows the clock: the first steps of a burst run at the full clock, then the power
    cap pulls the clock down and the step time goes up with it."""
    import datetime
    import torch
    eng = model.engine
    clocks = ClockSampler(gpu_id, period_ms=20)
    slots = [eng.alloc_slot() for _ in range(2)]
    model.step([(slots[0], prompt, [len(prompt) - 1])])                     # warm the path
    eng.free_slot(slots[0])
    torch.cuda.synchronize()
    time.sleep(1.0)                                                         # let the GPU rest: the burst starts cool
    clocks.start()
    time.sleep(0.1)
    rows, events = [], []
    t_wall0 = time.time()
    for i in range(40):
        s = eng.alloc_slot()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        model.step([(s, prompt, [len(prompt) - 1])])
        b.record()
        eng.free_slot(s)
        events.append((a, b))
    torch.cuda.synchronize()
    t_wall1 = time.time()
    clocks.stop()
    samples = []
    for l in clocks.lines:
        f = [x.strip() for x in l.split(",")]
        try:
            samples.append((datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp(), float(f[1]), float(f[7])))
        except (ValueError, IndexError):
            pass
    ms = [a.elapsed_time(b) for a, b in events]
    t = t_wall0
    print("step   ms     TFLOP/s   sm MHz   W      ms x GHz")
    for i, m in enumerate(ms):
        mid = t + m / 2e3
        near = min(samples, key=lambda s: abs(s[0] - mid)) if samples else (0, float("nan"), float("nan"))
        print(f"{i:3d}  {m:6.2f}  {flops / m / 1e9:8.0f}  {near[1]:7.0f}  {near[2]:5.0f}  {m * near[1] / 1e3:7.2f}")
        t += (t_wall1 - t_wall0) / len(ms)
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=32)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration's 36 "
                    "(layer sizes stay); the JSON names both numbers")
    ap.add_argument("--no-points", action="store_true", help="skip decoding at batch 1 and 64")
    ap.add_argument("--write-model", default=None, metavar="DIR",
                    help="with --impl reference: only write the model folder that arm uses (tied head, --layers of the 36) "
                         "to DIR and exit, for running baseline/_ref/bin/reference_runner by hand or under a profiler")
    ap.add_argument("--study", default=None, choices=["prefill-clocks"],
                    help="prefill-clocks: 40 prompt steps of 2,048 tokens back to back with the clock and the power "
                         "sampled every 20 ms; prints a table and no JSON line")
    args = ap.parse_args()

    if args.impl == "reference":
        if args.gpus != 1:
            print(json.dumps({"impl": "reference", "unavailable": "upstream runs on one GPU only"}))
            return 0
        if args.write_model:
            write_reference_model(args.write_model, args.layers or QWEN3_8B["num_hidden_layers"])
            print(f"wrote {args.write_model}")
            return 0
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported (nothing was run)")
        return 2

    import torch
    from garlic_inference_b200 import LanguageModel, Qwen3Config
    from garlic_inference_b200.ops import counters
    from garlic_inference_b200.sampling import SamplingParams

    K, W = args.steps, max(args.warmup, 3)
    n_layers = args.layers or QWEN3_8B["num_hidden_layers"]
    cfg = Qwen3Config(**{**QWEN3_8B, "num_hidden_layers": n_layers})
    pk = peaks()
    torch.cuda.set_device(0)
    props = torch.cuda.get_device_properties(0)
    gpu_id = "GPU-" + str(props.uuid) if getattr(props, "uuid", None) else "0"
    batches = [args.batch] + ([] if args.no_points else [1, 64])
    per_seq = -(-(CACHED + W + K + 8) // 64) * 64
    long_points = [] if args.no_points else [(8, 8192), (1, 32768)]          # (batch, cached tokens): longer contexts
    max_tokens = max([max(batches) * per_seq, -(-PREFILL_TOKENS // 64) * 64 * 2] +
                     [b * (-(-(c + W + K + 8) // 64) * 64) for b, c in long_points])
    model = LanguageModel.from_random(cfg, seed=0, device=0, dtype="bfloat16", max_tokens=max_tokens)
    eng, sampler = model.engine, model.sampler
    gen = torch.Generator().manual_seed(0)
    greedy = SamplingParams()

    def random_prompt(n):
        return torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()

    def fill(batch, cached=CACHED):
        """`batch` slots, each holding `cached` tokens after a real prefill; returns slots and next tokens."""
        slots, firsts = [], []
        for _ in range(batch):
            s = eng.alloc_slot()
            logits = model.step([(s, random_prompt(cached), [cached - 1])])
            firsts.append(sampler.sample(logits, greedy, [0], [0]))
            slots.append(s)
        return slots, torch.cat(firsts)

    def time_decode(batch, clocks=None, cached=CACHED):
        slots, toks = fill(batch, cached)
        for _ in range(W):
            toks = sampler.sample(eng.step_decode_device(slots, toks), greedy, slots, slots)
        torch.cuda.synchronize()
        launches0 = counters.launches
        if clocks:
            clocks.start()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(K):
            toks = sampler.sample(eng.step_decode_device(slots, toks), greedy, slots, slots)
        end.record()
        torch.cuda.synchronize()
        if clocks:
            clocks.stop()
        ms = start.elapsed_time(end)
        launched = counters.launches - launches0
        for s in slots:
            eng.free_slot(s)
        return batch * K / (ms / 1e3), ms / K, launched

    if args.study == "prefill-clocks":
        return study_prefill_clocks(model, random_prompt(PREFILL_TOKENS), gpu_id,
                                    prefill_flops(QWEN3_8B, n_layers, PREFILL_TOKENS))

    # ---- prefill of 2,048 tokens --------------------------------------------------------------
    prompt = random_prompt(PREFILL_TOKENS)
    times = []
    pre_clocks = ClockSampler(gpu_id, period_ms=20)
    pre_clocks.start()
    for i in range(3 + 5):
        s = eng.alloc_slot()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        model.step([(s, prompt, [PREFILL_TOKENS - 1])])
        b.record()
        torch.cuda.synchronize()
        eng.free_slot(s)
        if i >= 3:
            times.append(a.elapsed_time(b))
    pre_clocks.stop()
    pre_ms = statistics.median(times)
    pre_flops = prefill_flops(QWEN3_8B, n_layers, PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / (pre_ms / 1e3), "tokens": PREFILL_TOKENS, "ms": pre_ms,
               "frac": pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12),
               "frac_of_sustained": (pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12)
                                     if pk.get("bf16_tflops_sustained") else None),
               "sm_mhz": pre_clocks.summary().get("sm_mhz")}

    # ---- decoding, timed on the device ----------------------------------------------------------
    clocks = ClockSampler(gpu_id)
    value, ms_per_step, launched = time_decode(args.batch, clocks)
    avg_ctx = CACHED + W + (K + 1) / 2
    total_b, weight_b, kv_b = decode_step_bytes(QWEN3_8B, n_layers, args.batch, avg_ctx)
    achieved = total_b / (ms_per_step / 1e3) / 1e9
    points = {}
    if not args.no_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = time_decode(b)[0]
        for b, c in long_points:                         # the same through the engine at longer contexts, with the
            tok_s, ms, _ = time_decode(b, cached=c)      # fraction of the measured copy bandwidth the step's bytes reach
            step_b = decode_step_bytes(QWEN3_8B, n_layers, b, c + W + (K + 1) / 2)[0]
            points[f"decode_b{b}_ctx{c}"] = tok_s
            points[f"decode_b{b}_ctx{c}_hbm_frac"] = step_b / (ms / 1e3) / 1e9 / pk["hbm_gbs"]

    # ---- the same through the entry point: host ids in, host ids out, every step ------------------
    # W + K + 1 tokens per request; the clock runs over the last K steps (the W before them are the warm-up,
    # as in the device-timed loop above), read from the loop's own record of when each step's tokens arrived
    prompts = [random_prompt(CACHED) for _ in range(args.batch)]
    model.generate(prompts[:1], max_new_tokens=4)                           # warm the path
    up0 = eng.bytes_uploaded
    e2e_clocks = ClockSampler(gpu_id, period_ms=20)
    wall_minus_perf = time.time() - time.perf_counter()
    e2e_clocks.start()
    out = model.generate(prompts, max_new_tokens=W + K + 1)
    e2e_clocks.stop()
    st = model.last_stats
    assert all(len(o) == W + K + 1 for o in out) and len(st.step_times) == W + K + 1
    e2e_seconds = st.step_times[-1] - st.step_times[-1 - K]
    # the clock during the timed steps of this run (its prompt step of batch x 2,048 tokens comes right before them),
    # so that ms x MHz of the two decode figures can be compared
    e2e_clk = e2e_clocks.summary(since=st.step_times[-1 - K] + wall_minus_perf, until=st.step_times[-1] + wall_minus_perf)
    e2e = {"value": args.batch * K / e2e_seconds, "unit": "tokens/s",
           "h2d_bytes_per_step": (eng.bytes_uploaded - up0) / st.steps,
           "d2h_bytes_per_step": 4 * args.batch, "ms_per_step": 1e3 * e2e_seconds / K,
           "sm_mhz": e2e_clk.get("sm_mhz"), "watts": e2e_clk.get("watts")}
    page_size = eng.cache.page_size
    workloads = {} if args.no_points else larger_workloads(model, pk, gpu_id)

    line = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen3-8B layer sizes, {CACHED} cached tokens per sequence)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02) made on the GPU, uniform random token ids",
        "config": {"model": "Qwen3-8B layer sizes", "global_batch": args.batch, "seq_len": CONTEXT,
                   "cached_tokens": CACHED, "parallelism": "none (1 GPU)", "layers_run": n_layers,
                   "layers_config": QWEN3_8B["num_hidden_layers"], "hidden_size": 4096, "n_heads": 32,
                   "n_kv_heads": 8, "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936,
                   "page_size": page_size, "sampling": "greedy on the device",
                   "l2": "inputs exceed L2: a step reads %.1f GB of weights" % (weight_b / 1e9)},
        "clocks": clocks.summary(),
        "e2e": e2e,
        "gpu_launches": launched,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "bytes_per_step": total_b, "peaks": pk["source"]},
        "points": points,
        "workloads": workloads,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
