"""The command line: `runner MODEL_DIR`, in upstream's manner.

Upstream's `runner [MODEL DIR]` asks for one prompt on standard input, runs
601 greedy steps and prints the text, then `Time:` in milliseconds and
`Tok/s:` with the prompt's step left out of the clock (inference.cpp:29-35,
111-113, 161-177).  This one keeps the positional model folder, the prompt on
standard input and the two closing lines.  It has no tokenizer: prompts are
token ids (one prompt a line, ids separated by spaces or commas) and so is
the output.  What upstream fixes in code is an option here.
"""
from __future__ import annotations

import argparse
import re
import sys


def parse_ids(text: str) -> list[int]:
    parts = [p for p in re.split(r"[,\s]+", text.strip()) if p]
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit(f"a prompt is a list of token ids; cannot read {text.strip()!r}") from None


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="runner", description="generate token ids with a model folder on one B200")
    ap.add_argument("model_dir", metavar="MODEL_DIR",
                    help="folder with config.json and model.safetensors (with --random-weights: a config.json "
                         "or a folder that holds one; no weights are read)")
    ap.add_argument("--prompt-ids", action="append", default=None,
                    help="a prompt as token ids '1,2,3' (repeat for a batch); default: read prompts from stdin")
    ap.add_argument("--prompt-file", default=None, help="a file with one prompt (token ids) per line")
    ap.add_argument("--random-weights", action="store_true",
                    help="random weights of the configuration's sizes, made on the device")
    ap.add_argument("--weights-seed", type=int, default=0, help="seed of --random-weights")
    ap.add_argument("--max-new-tokens", type=int, default=600, help="tokens to generate per prompt (upstream: 600)")
    ap.add_argument("--temperature", type=float, default=0.0, help="0 = greedy (upstream's only mode)")
    ap.add_argument("--seed", type=int, default=0, help="seed of temperature sampling")
    ap.add_argument("--stop-ids", default=None, help="token ids that end a request, '7,8' (default: the folder's "
                    "generation_config.json eos_token_id, else none)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-tokens", type=int, default=None,
                    help="cache size in tokens (default: what the given prompts need)")
    ap.add_argument("--max-batch", type=int, default=None, help="most requests in one batch")
    ap.add_argument("--max-slots", type=int, default=None,
                    help="most requests the cache can hold at once (default: one per 64 tokens of the cache)")
    ap.add_argument("--print-logits", type=int, default=0, metavar="N",
                    help="before generating, run each prompt once and print the N largest logits (id:value) at its "
                         "last position, for comparing numbers with another implementation")
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--device", type=int, default=0)
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.prompt_ids or args.prompt_file:
        prompts = [parse_ids(p) for p in args.prompt_ids or []]
        if args.prompt_file:
            with open(args.prompt_file) as f:
                prompts += [parse_ids(line) for line in f if line.strip()]
    else:
        if sys.stdin.isatty():
            print("Ask the model something (token ids): ", end="", flush=True)
            prompts = [parse_ids(sys.stdin.readline())]
        else:
            prompts = [parse_ids(line) for line in sys.stdin if line.strip()]
    prompts = [p for p in prompts if p]
    if not prompts:
        raise SystemExit("no prompt given")

    from .engine import AutoModel
    from .engine.generate import tokens_held
    from .config import load_config
    max_pos = load_config(args.model_dir).max_position_embeddings
    need = sum(tokens_held(len(p), args.max_new_tokens, max_pos) for p in prompts[:args.max_batch or len(prompts)])
    if args.random_weights:
        model = AutoModel.from_random(load_config(args.model_dir), seed=args.weights_seed, device=args.device,
                                      dtype=args.dtype, max_tokens=args.max_tokens or need, page_size=args.page_size,
                                      max_slots=args.max_slots)
    else:
        model = AutoModel.from_pretrained(args.model_dir, device=args.device, dtype=args.dtype,
                                          max_tokens=args.max_tokens or need, page_size=args.page_size,
                                          max_slots=args.max_slots)
    if args.print_logits > 0:
        for i, p in enumerate(prompts):
            slot = model.alloc_slot()
            row = model.step([(slot, p, [len(p) - 1])])[0]
            model.free_slot(slot)
            top = row.topk(min(args.print_logits, row.numel()))
            print(f"Logits {i}: " + " ".join(f"{int(t)}:{float(v):.6g}" for v, t in zip(top.values.tolist(), top.indices.tolist())))
    stop = None if args.stop_ids is None else parse_ids(args.stop_ids)
    out = model.generate(prompts, max_new_tokens=args.max_new_tokens, temperature=args.temperature,
                         seed=args.seed, stop_token_ids=stop, max_batch=args.max_batch)
    for ids in out:
        print(" ".join(str(t) for t in ids))
    st = model.last_stats
    decoded = st.new_tokens - len(prompts)                       # each request's first token is the prompt step's
    print(f"Time: {st.decode_seconds * 1000.0:.0f}")
    print(f"Tok/s: {decoded / st.decode_seconds if st.decode_seconds > 0 and decoded > 0 else 0.0:.1f}")
    print(f"Prefill tok/s: {st.prompt_tokens / st.prefill_seconds if st.prefill_seconds > 0 else 0.0:.1f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
